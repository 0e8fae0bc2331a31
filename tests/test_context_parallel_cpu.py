"""Context-parallel attention (contiguous / zigzag / ring), SSD scan (two-pass and serial) and conv1d halo on gloo
ranks against the single-process results, forward and backward."""
import os
import subprocess
import sys

import pytest
import torch

from sneppx_alg_b200.parallel import context as cp


def test_zigzag_roundtrip_and_merge():
    x = torch.arange(2 * 24 * 3, dtype=torch.float32).view(2, 24, 3)
    shards = [cp.zigzag_split(x, 3, r) for r in range(3)]
    assert shards[0].shape == (2, 8, 3) and torch.equal(shards[0][:, :4], x[:, :4]) and torch.equal(shards[0][:, 4:], x[:, 20:])
    assert torch.equal(cp.zigzag_merge(shards), x)


def test_merge_attention_blocks_equals_joint_softmax():
    from sneppx_alg_b200.ops import functional as F_
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 5, 2, 8), torch.randn(1, 12, 2, 8), torch.randn(1, 12, 2, 8)
    o1, l1 = F_.attention_with_lse(q, k[:, :7], v[:, :7], causal=False)
    o2, l2 = F_.attention_with_lse(q, k[:, 7:], v[:, 7:], causal=False)
    o, _ = cp.merge_attention_blocks(o1.float(), l1, o2, l2)
    assert torch.allclose(o, F_.attention_reference(q, k, v, causal=False), atol=1e-5)


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_ranks(world):
    script = os.path.join(os.path.dirname(__file__), "mp_cp_check.py")
    port = 29620 + world + (os.getpid() % 200)
    r = subprocess.run([sys.executable, script, str(world), str(port)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
