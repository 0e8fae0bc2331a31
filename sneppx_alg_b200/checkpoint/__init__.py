"""checkpoint sub-package."""
