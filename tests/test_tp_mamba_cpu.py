"""Tensor-parallel Mamba-2 block and language model on gloo ranks against their unsharded forms."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("script,marker,port", [("mp_tp_mamba_check.py", "TP_MAMBA_OK", 29750),
                                                ("mp_tp_mamba_model_check.py", "TP_MAMBA_MODEL_OK", 29760)])
def test_tp_mamba_two_ranks(script, marker, port):
    r = subprocess.run([sys.executable, os.path.join(HERE, script), "2", str(port + os.getpid() % 7)], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0 and marker in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_tp_dp_engine_four_ranks():
    r = subprocess.run([sys.executable, os.path.join(HERE, "mp_tp_dp_engine_check.py"), "4", str(29770 + os.getpid() % 7)],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "TP_DP_ENGINE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_tp_mamba_benchmark_runs_on_gloo():
    import json
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr", "127.0.0.1",
           "--master-port", str(29790 + os.getpid() % 7), "-m", "sneppx_alg_b200.benchmarks.tp_mamba", "--tp", "2", "--model", "tiny",
           "--seq", "64", "--device", "cpu", "--steps", "2", "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=os.path.dirname(HERE))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["config"]["parallelism"] == "tp2xdp2" and line["value"] > 0 and line["last_loss"] < 6.0
