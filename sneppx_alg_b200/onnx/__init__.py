"""onnx sub-package."""
