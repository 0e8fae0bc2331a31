"""``jit``: trace / grad / vmap / jacobian / hessian (the reference's ``jit.py``) and graph capture.

There is no tracing compiler here: ``trace`` captures the function's kernel launches into a CUDA graph (static
shapes, static input buffers) and replays it, which removes launch overhead from launch-bound loops; on CPU tensors it
returns the function unchanged.  The transforms are ``torch.func``."""
from __future__ import annotations

import torch
from torch import func as _func

grad = _func.grad
value_and_grad = _func.grad_and_value
vmap = _func.vmap
jacobian = _func.jacrev
jacfwd = _func.jacfwd
hessian = _func.hessian
vjp, jvp = _func.vjp, _func.jvp


class GraphedCallable:
    """A function captured once into a CUDA graph.  Inputs are copied into the captured static buffers before each
    replay; outputs alias the captured output buffers (clone them to keep a result across calls)."""

    def __init__(self, fn, example_inputs, warmup=3, pool=None):
        assert all(t.is_cuda for t in example_inputs), "CUDA graph capture needs CUDA tensors"
        self.static_in = [t.clone() for t in example_inputs]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(warmup):
                fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(s)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool), torch.no_grad():
            self.static_out = fn(*self.static_in)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_in, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        self.graph.replay()
        return self.static_out


def trace(fn, *example_inputs, warmup=3):
    if example_inputs and all(torch.is_tensor(t) and t.is_cuda for t in example_inputs):
        return GraphedCallable(fn, example_inputs, warmup)
    return fn
