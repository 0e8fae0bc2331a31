"""Fused ZeRO path on 2 GPUs against the torch.distributed library path (skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("stage,mode", [(1, "p2p"), (3, "p2p"), (3, "nvls"), (3, "slots")])
def test_fused_zero_two_gpus(stage, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29600 + stage + {"nvls": 4, "slots": 6}.get(mode, 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_zero_check.py"), str(stage), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-1500:]


def test_fused_tensor_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29611", os.path.join(HERE, "mp_tp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-1500:]


def test_fused_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29621", os.path.join(HERE, "mp_ep_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-1500:]


def test_context_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "mp_cp_gpu_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "CP_GPU_OK" in r.stdout, r.stdout[-4000:] + r.stderr[-1500:]


def test_tensor_parallel_mamba_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29641", os.path.join(HERE, "mp_tp_mamba_gpu_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-1500:]


def test_pipeline_ulysses_hierarchical_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29651", os.path.join(HERE, "mp_pp_sp_gpu_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0 and "PP_SP_GPU_OK" in r.stdout, r.stdout[-4000:] + r.stderr[-1500:]


def test_tensor_parallel_serving_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29661", os.path.join(HERE, "mp_tp_serving_gpu_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-1500:]
