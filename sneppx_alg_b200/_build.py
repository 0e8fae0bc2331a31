"""Builds and loads the native libraries of the framework, in-tree.

Two shared objects are produced under ``sneppx_alg_b200/lib``:

* ``libsneppx_b200.so``  - every CUDA kernel (``csrc/*.cu``), compiled by ``nvcc`` for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); exported through a C ABI (``csrc/sx_api.h``) and
  called from Python with ``ctypes``.
* ``libsneppx_host.so``  - the host-side C++ runtime (``csrc/host/*.cpp``): checkpoint container,
  TCP ring all-reduce, heartbeat, model factory, serving batch core, tokenizer, edge runtime.

A content hash of the sources is stored beside each library; ``load_*`` rebuilds when the hash no
longer matches and a compiler is available, and fails loudly otherwise.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread", "-Wall", "-Wno-unused-function"]

_lock = threading.Lock()
_cuda_lib = None
_host_lib = None


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _hash_files(files, extra=()) -> str:
    h = hashlib.sha256()
    for f in sorted(files):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def cuda_sources():
    return sorted(CSRC.glob("*.cu"))


def cuda_headers():
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def host_sources():
    return sorted((CSRC / "host").glob("*.cpp"))


def host_headers():
    return sorted((CSRC / "host").glob("*.h")) + sorted((CSRC / "host").glob("*.hpp")) + [CSRC / "conv2d_bwd_body.h", CSRC / "npe_body.h"]


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(map(str, cmd)) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def _compile_objects(compiler, flags, sources, headers, tag, verbose):
    OBJDIR.mkdir(parents=True, exist_ok=True)
    hdr_hash = _hash_files(headers, flags)
    jobs = []
    objs = []
    for src in sources:
        obj = OBJDIR / f"{tag}_{src.stem}.o"
        stamp = OBJDIR / f"{tag}_{src.stem}.hash"
        want = _hash_files([src], [hdr_hash])
        objs.append(obj)
        if obj.exists() and stamp.exists() and stamp.read_text() == want:
            continue
        jobs.append((src, obj, stamp, want))

    def one(job):
        src, obj, stamp, want = job
        out = _run([compiler, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
        stamp.write_text(want)
        if verbose:
            print(f"[sneppx build] {src.name}", file=sys.stderr)
            if out.strip():
                print(out, file=sys.stderr)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(one, jobs))
    return objs


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libsneppx_b200.so``."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    lib = LIBDIR / "libsneppx_b200.so"
    stamp = LIBDIR / "libsneppx_b200.hash"
    want = _hash_files(cuda_sources() + cuda_headers(), NVCC_FLAGS)
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == want:
        return lib
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libsneppx_b200.so")
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose else [])
    objs = _compile_objects(nvcc, flags, cuda_sources(), cuda_headers(), "cu", verbose)
    _run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"])
    stamp.write_text(want)
    return lib


def build_host(force: bool = False, verbose: bool = False) -> Path:
    """Compile the host C++ runtime into ``libsneppx_host.so``."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    lib = LIBDIR / "libsneppx_host.so"
    stamp = LIBDIR / "libsneppx_host.hash"
    srcs = host_sources()
    want = _hash_files(srcs + host_headers(), CXX_FLAGS)
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == want:
        return lib
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found: cannot build libsneppx_host.so")
    objs = _compile_objects(cxx, CXX_FLAGS + ["-I", str(CSRC / "host")], srcs, host_headers(), "host", verbose)
    _run([cxx, "-shared", "-o", str(lib), *map(str, objs), "-pthread"])
    stamp.write_text(want)
    return lib


SANITIZE_FLAGS = ["-O1", "-g", "-std=c++17", "-fPIC", "-pthread", "-fsanitize=address,undefined", "-fno-omit-frame-pointer"]


def build_host_sanitized(verbose: bool = False, kind: str = "address") -> Path:
    """Sanitizer build of the host runtime. ``kind="address"``: AddressSanitizer + UndefinedBehaviorSanitizer
    (``libsneppx_host_asan.so``); ``kind="thread"``: ThreadSanitizer (``libsneppx_host_tsan.so``). Run the host-side
    tests against it with ``LD_PRELOAD=$(g++ -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0
    SX_HOST_LIB=<path> python -m pytest ...`` (``libtsan.so`` and ``TSAN_OPTIONS=report_signal_unsafe=0`` for the thread
    build); the reference's ``scripts/run_sanitizers.sh`` does the same for its C tests."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    tag, san = ("tsan", "thread") if kind == "thread" else ("asan", "address,undefined")
    lib = LIBDIR / f"libsneppx_host_{tag}.so"
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found")
    srcs = host_sources()
    flags = [f if not f.startswith("-fsanitize=") else f"-fsanitize={san}" for f in SANITIZE_FLAGS]
    objs = _compile_objects(cxx, flags + ["-I", str(CSRC / "host")], srcs, host_headers(), f"host_{tag}", verbose)
    _run([cxx, "-shared", "-o", str(lib), *map(str, objs), "-pthread", f"-fsanitize={san}"])
    return lib


def build_all(force: bool = False, verbose: bool = False):
    return build_cuda(force, verbose), build_host(force, verbose)


def load_cuda() -> ctypes.CDLL:
    """Return the CUDA kernel library, building it first when the sources changed."""
    global _cuda_lib
    with _lock:
        if _cuda_lib is None:
            lib = LIBDIR / "libsneppx_b200.so"
            try:
                lib = build_cuda()
            except RuntimeError as e:
                if not lib.exists():
                    raise
                import warnings
                warnings.warn(f"sneppx_alg_b200: rebuilding the CUDA library FAILED ({e}); loading the existing "
                              f"{lib.name}, which was built from OLDER sources", RuntimeWarning, stacklevel=2)
                print(f"[sneppx_alg_b200] WARNING: stale {lib} in use, rebuild failed: {e}", file=sys.stderr, flush=True)
            _cuda_lib = ctypes.CDLL(str(lib), mode=ctypes.RTLD_GLOBAL)
        return _cuda_lib


def load_host() -> ctypes.CDLL:
    global _host_lib
    with _lock:
        if _host_lib is None:
            override = os.environ.get("SX_HOST_LIB")   # e.g. the sanitizer build from build_host_sanitized()
            if override:
                _host_lib = ctypes.CDLL(override)
                return _host_lib
            lib = LIBDIR / "libsneppx_host.so"
            try:
                lib = build_host()
            except RuntimeError:
                if not lib.exists():
                    raise
            _host_lib = ctypes.CDLL(str(lib))
        return _host_lib


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
