"""The allocation-free gradient-norm entry point, called through its exported C symbol.

Callers that cannot reserve device memory (a fixed memory plan, a capture region, a no-new-allocations
policy) use ``sx_grad_sumsq_noalloc``; it must give what the regular entry point ``sx_grad_sumsq`` gives (that one
works in a buffer its caller allocates). It is checked on repeated calls because every call of the allocation-free
entry point works in the same built-in per-device scratch array, which still holds the previous call's data.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from sneppx_alg_b200 import _build
    lib = _build.load_cuda()
    fn = lib.sx_grad_sumsq_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]
    ref = lib.sx_grad_sumsq
    ref.restype = C.c_int
    ref.argtypes = [C.c_void_p, C.c_int, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                    C.c_float, C.c_void_p]
    return fn, ref


def test_noalloc_matches_regular_entry_point_twice():
    fn, ref = _lib()
    torch.manual_seed(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    partials = torch.empty(1024, dtype=torch.float32, device="cuda")
    # two calls in a row with different sizes and dtypes: the second must not see the first one's partials
    for n, dtype, max_norm in ((3_000_017, torch.bfloat16, 1.0), (70_001, torch.float32, 0.0)):
        g = torch.randn(n, device="cuda").to(dtype)
        out = torch.full((3,), -1.0, device="cuda")
        out_ref = torch.full((3,), -1.0, device="cuda")
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        flag_ref = torch.zeros(1, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(g.data_ptr(), int(dtype == torch.bfloat16), n, out.data_ptr(), flag.data_ptr(), max_norm, stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        rc = ref(g.data_ptr(), int(dtype == torch.bfloat16), n, partials.data_ptr(), out_ref.data_ptr(),
                 flag_ref.data_ptr(), 0, 1, max_norm, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(out, out_ref, rtol=1e-5, atol=1e-6), (out, out_ref)
        exact = g.double().pow(2).sum().item()
        assert abs(out[0].item() - exact) < 1e-3 * exact
        assert flag.item() == flag_ref.item() == 0


def test_noalloc_rejects_bad_sizes():
    fn, _ = _lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.zeros(3, device="cuda")
    g = torch.zeros(8, device="cuda")
    assert fn(g.data_ptr(), 0, (1 << 33) + 1, out.data_ptr(), None, 0.0, stream) == -40
    assert fn(g.data_ptr(), 0, 0, out.data_ptr(), None, 0.0, stream) == -41
