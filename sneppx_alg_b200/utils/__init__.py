"""utils sub-package."""
