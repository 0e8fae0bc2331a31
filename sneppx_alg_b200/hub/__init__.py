"""hub sub-package."""
