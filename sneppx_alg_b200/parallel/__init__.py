"""parallel sub-package."""
