"""The header-only C++ interface compiles against the host library and interoperates with the Python side."""
import os
import shutil
import subprocess

import pytest

from sneppx_alg_b200 import _build

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_program_uses_checkpoint_tokenizer_factory_and_kem(tmp_path):
    lib = _build.build_host() if hasattr(_build, "build_host") else None
    libdir = os.path.dirname(str(lib)) if lib else str(_build.LIBDIR)
    inc = os.path.join(os.path.dirname(_build.__file__), "csrc", "host", "include")
    exe = str(tmp_path / "check")
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", inc, os.path.join(HERE, "data", "cpp_api_check.cpp"),
                        "-L", libdir, "-lsneppx_host", f"-Wl,-rpath,{libdir}", "-o", exe], capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "CPP_API_OK" in r.stdout, (r.returncode, r.stdout, r.stderr)
    assert "sha256 ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad" in r.stdout

    # what the C++ program wrote is readable from Python, and the reverse
    from sneppx_alg_b200.checkpoint.sneppx_format import load_tensors
    tensors, meta = load_tensors(str(tmp_path / "from_cpp.sneppx"))
    vals = list(tensors.values()) if isinstance(tensors, dict) else list(tensors)
    assert vals[0].tolist() == [[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]] and vals[1].tolist() == [0, 10, 20, 30]
    from sneppx_alg_b200.security import crypto
    ek, dk = crypto.mlkem_keygen(768, seed=bytes(range(64)))
    ss, ct = crypto.mlkem_encaps(ek, 768, message=bytes(range(200, 232)))
    assert crypto.mlkem_decaps(dk, ct, 768) == ss


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_example_builds_and_runs(tmp_path):
    lib = _build.build_host() if hasattr(_build, "build_host") else None
    libdir = os.path.dirname(str(lib)) if lib else str(_build.LIBDIR)
    inc = os.path.join(os.path.dirname(_build.__file__), "csrc", "host", "include")
    src = os.path.join(os.path.dirname(HERE), "examples", "cpp", "host_runtime_demo.cpp")
    exe = str(tmp_path / "demo")
    r = subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", inc, src, "-L", libdir, "-lsneppx_host",
                        f"-Wl,-rpath,{libdir}", "-o", exe], capture_output=True, text=True, timeout=200)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "HOST_RUNTIME_DEMO_OK" in r.stdout and "round trip exact" in r.stdout, (r.returncode, r.stdout, r.stderr)
    # the files it wrote open from Python: same tokenizer, same tensors
    from sneppx_alg_b200.checkpoint.sneppx_format import load_tensors
    from sneppx_alg_b200.utils.host import BPETokenizer
    tensors, meta = load_tensors(str(tmp_path / "demo.sneppx"))
    vals = list(tensors.values())
    tok = BPETokenizer()
    tok.load(str(tmp_path / "demo.tok"))
    assert meta["tokenizer"] == "demo.tok" and vals[0].shape[1] == 8
    assert tok.decode(vals[1].tolist()) == "the lazy fox sleeps over the quick dog."
