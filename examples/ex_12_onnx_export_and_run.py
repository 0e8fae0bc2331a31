"""Export a feed-forward module to ONNX with the built-in toolkit (no onnx package needed), check and optimise the
graph, run it with the NumPy executor, quantise it (QDQ) and compare all three with the PyTorch module."""
from _common import seed  # first: makes the package importable from a checkout
import os
import tempfile

import numpy as np
import torch

from sneppx.onnx import toolkit as onnx


def main() -> dict:
    seed(10)
    module = torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.GELU(), torch.nn.LayerNorm(32), torch.nn.Linear(32, 4)).eval()
    x = torch.randn(5, 16)
    with torch.no_grad():
        want = module(x).numpy()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "mlp.onnx")
        model = onnx.export_module(module, x, path)
        size = os.path.getsize(path)
        loaded = onnx.Model.load(path)
    problems = onnx.check_model(loaded)
    got = list(onnx.run_model(loaded, {"input": x.numpy()}).values())[0]
    optimised = onnx.optimize(loaded)
    got_opt = list(onnx.run_model(optimised, {"input": x.numpy()}).values())[0]
    quantised = onnx.quantize_qdq(loaded)
    got_q = list(onnx.run_model(quantised, {"input": x.numpy()}).values())[0]
    out = {"file_bytes": size, "nodes": (len(loaded.graph.nodes), len(optimised.graph.nodes), len(quantised.graph.nodes)),
           "problems": problems, "max_error": float(np.abs(got - want).max()), "max_error_optimised": float(np.abs(got_opt - want).max()),
           "max_error_qdq": float(np.abs(got_q - want).max()), "shapes": onnx.infer_shapes(loaded, {"input": (5, 16)})}
    print(f"{size} bytes, nodes exported / optimised / quantised = {out['nodes']}, checker problems: {problems or 'none'}")
    print(f"max |onnx - torch| = {out['max_error']:.2e} (optimised {out['max_error_optimised']:.2e}, int8 QDQ {out['max_error_qdq']:.3f})")
    return out


if __name__ == "__main__":
    main()
