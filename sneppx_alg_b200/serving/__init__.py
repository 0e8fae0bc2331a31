"""serving sub-package."""
