"""training sub-package."""
