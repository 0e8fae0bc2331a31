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
