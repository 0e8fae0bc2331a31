"""optim sub-package."""
