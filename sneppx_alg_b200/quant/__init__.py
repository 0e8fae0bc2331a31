"""quant sub-package."""
