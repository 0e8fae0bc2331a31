"""security sub-package."""
