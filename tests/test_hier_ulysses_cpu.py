"""Hierarchical all-reduce and Ulysses sequence parallelism on gloo ranks."""
import os
import subprocess
import sys


def test_hierarchical_all_reduce_and_ulysses_attention_on_four_ranks():
    script = os.path.join(os.path.dirname(__file__), "mp_hier_ulysses_check.py")
    port = 29750 + (os.getpid() % 200)
    r = subprocess.run([sys.executable, script, str(port)], capture_output=True, text=True, timeout=280)
    assert r.returncode == 0 and "HIER_ULYSSES_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
