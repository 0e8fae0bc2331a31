"""Bounded device waits: a barrier whose peer never signals gives up after its limit, reports through the status
word, and leaves the context usable. The 'peer' is a second signal pad on the same GPU that nothing writes; no trap,
failing assert or bad address is involved."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_barrier_wait_times_out_and_context_survives():
    from sneppx_alg_b200 import ops
    from sneppx_alg_b200.ops import _lib
    from sneppx_alg_b200.parallel.symm import PAD_WORDS, SxPeers
    dev = torch.device("cuda", 0)
    pads = [torch.zeros(PAD_WORDS, dtype=torch.int32, device=dev) for _ in range(2)]
    p = SxPeers()
    for r in range(2):
        p.pad[r] = pads[r].data_ptr()
        p.buf[r] = pads[r].data_ptr()
    p.rank, p.world, p.timeout_ns = 0, 2, 300_000_000            # 0.3 s
    status = _lib.status_word(dev)
    status.zero_()
    _lib.call("sx_peer_barrier", C.byref(p), C.c_int(5), C.c_uint(1), C.c_void_p(status.data_ptr()), _lib.stream())
    torch.cuda.synchronize()
    assert int(status[0]) != 0                                    # the wait ran out and said so
    with pytest.raises(ops.KernelTimeout):
        ops.check_status(dev)
    assert int(status[0]) == 0                                    # check_status reset the word
    # rank 0 did signal its peer before waiting
    assert int(pads[1][5 * 16 + 0]) == 1
    # the context is intact: an ordinary kernel still runs and gives the right answer
    a = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    out = ops.gemm(a, a)
    torch.cuda.synchronize()
    ref = a.float() @ a.float().T
    assert (out.float() - ref).abs().max() / ref.abs().max() < 2e-2
