"""`.sneppx` checkpoint files from Python: ``CheckpointWriter`` / ``CheckpointReader`` / ``validate_checkpoint`` with
the reference's method names (interface_bindings/checkpoint.py:96-196) on top of the C++ container
(``csrc/host/checkpoint.cpp``); tensor-level helpers ``save_tensors`` / ``load_tensors`` that carry names, dtypes and
shard information in the metadata JSON (the container itself only knows shapes and byte sizes)."""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import _build

MAGIC_LO, MAGIC_HI, VERSION = 0x41524958, 0x434B5054, 1
DTYPE_CODES = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3, torch.int32: 4, torch.int64: 5,
               torch.uint8: 6, torch.float8_e4m3fn: 7, torch.int8: 8, torch.bool: 9, torch.int16: 10}
CODE_DTYPES = {v: k for k, v in DTYPE_CODES.items()}


def _lib():
    L = _build.load_host()
    if not getattr(L, "_ckpt_ready", False):
        L.sx_ckpt_open.restype = C.c_void_p
        L.sx_ckpt_open.argtypes = [C.c_char_p]
        L.sx_ckpt_metadata.restype = C.c_char_p
        L.sx_ckpt_metadata.argtypes = [C.c_void_p]
        L.sx_ckpt_total_size.restype = C.c_ulonglong
        for f in ("sx_ckpt_num_tensors", "sx_ckpt_close", "sx_ckpt_total_size"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_ckpt_tensor_info.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sx_ckpt_read_tensor.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.sx_ckpt_saver_create.restype = C.c_void_p
        L.sx_ckpt_saver_submit.argtypes = [C.c_void_p, C.c_char_p, C.c_int] + [C.c_void_p] * 5 + [C.c_char_p]
        L.sx_ckpt_saver_wait.argtypes = [C.c_void_p]
        L.sx_ckpt_saver_destroy.argtypes = [C.c_void_p]
        L._ckpt_ready = True
    return L


def _pack_args(parts: List[Tuple[bytes, tuple, int, tuple]]):
    n = len(parts)
    shapes = (C.c_uint64 * (8 * n))()
    strides = (C.c_uint64 * (8 * n))()
    ndims = (C.c_uint32 * n)()
    dtypes = (C.c_uint32 * n)()
    nbytes = (C.c_uint64 * n)()
    ptrs = (C.c_void_p * n)()
    keep = []
    for i, (data, shape, dtype, stride) in enumerate(parts):
        for d, s in enumerate(shape):
            shapes[8 * i + d] = s
        for d, s in enumerate(stride):
            strides[8 * i + d] = s
        ndims[i], dtypes[i], nbytes[i] = len(shape), dtype, len(data)
        buf = C.create_string_buffer(data, len(data)) if not isinstance(data, (np.ndarray,)) else data
        keep.append(buf)
        ptrs[i] = C.cast(buf, C.c_void_p) if not isinstance(buf, np.ndarray) else buf.ctypes.data
    return n, shapes, ndims, dtypes, ptrs, nbytes, strides, keep


class CheckpointWriter:
    def __init__(self, path: str):
        self.path = path
        self._parts: List[Tuple[bytes, tuple, int, tuple]] = []
        self._meta: dict = {}

    def write_tensor(self, data: bytes, shape: tuple = (), dtype: int = 0, strides: tuple = ()):
        self._parts.append((bytes(data), tuple(shape), int(dtype), tuple(strides)))

    def write_metadata(self, meta: dict):
        self._meta.update(meta)

    def close(self):
        n, shapes, ndims, dtypes, ptrs, nbytes, strides, keep = _pack_args(self._parts)
        meta = json.dumps(self._meta).encode("utf-8") if self._meta else None
        rc = _lib().sx_ckpt_write(self.path.encode(), n, shapes, ndims, dtypes, ptrs, nbytes, meta, strides)
        if rc != 0:
            raise IOError(f"writing {self.path} failed ({rc})")

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if exc[0] is None:
            self.close()


class CheckpointReader:
    def __init__(self, path: str):
        self.path = path
        self._h = _lib().sx_ckpt_open(path.encode())
        if not self._h:
            raise ValueError(f"Invalid or unreadable checkpoint at {path}")
        self.num_tensors = _lib().sx_ckpt_num_tensors(self._h)

    def tensor_info(self, idx: int):
        shape = (C.c_uint64 * 8)()
        ndim, dtype, nbytes = C.c_uint32(), C.c_uint32(), C.c_uint64()
        if _lib().sx_ckpt_tensor_info(self._h, idx, shape, C.byref(ndim), C.byref(dtype), C.byref(nbytes)) != 0:
            raise IndexError(idx)
        return tuple(shape[: ndim.value]), dtype.value, nbytes.value

    def read_tensor(self, idx: int) -> bytes:
        _, _, nbytes = self.tensor_info(idx)
        buf = C.create_string_buffer(nbytes)
        if _lib().sx_ckpt_read_tensor(self._h, idx, buf) != 0:
            raise IOError(f"reading tensor {idx} of {self.path} failed")
        return buf.raw

    def read_metadata(self) -> dict:
        m = _lib().sx_ckpt_metadata(self._h)
        return json.loads(m.decode("utf-8")) if m else {}

    def close(self):
        if self._h:
            _lib().sx_ckpt_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def validate_checkpoint(path: str) -> bool:
    try:
        with CheckpointReader(path) as r:
            total = os.path.getsize(path)
            if _lib().sx_ckpt_total_size(r._h) != total:
                return False
            for i in range(r.num_tensors):
                r.tensor_info(i)
            r.read_metadata()
        return True
    except Exception:  # noqa: BLE001
        return False


# ----------------------------------------------------------------------------- tensor-level helpers
def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().cpu().contiguous()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def save_tensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None, saver=None):
    """Write named tensors (any dtype) in dict order; names / dtypes / shapes go into the metadata JSON."""
    names = list(tensors)
    meta = dict(metadata or {})
    meta["tensor_names"] = names
    meta["tensor_shapes"] = [list(tensors[n].shape) for n in names]
    meta["tensor_dtypes"] = [str(tensors[n].dtype).replace("torch.", "") for n in names]
    parts = [(_to_bytes(tensors[n]), tuple(tensors[n].shape), DTYPE_CODES.get(tensors[n].dtype, 6), ()) for n in names]
    if saver is not None:
        return saver.submit(path, parts, meta)
    w = CheckpointWriter(path)
    w._parts, w._meta = parts, meta
    w.close()


def load_tensors(path: str, device="cpu") -> Tuple[Dict[str, torch.Tensor], dict]:
    out = {}
    with CheckpointReader(path) as r:
        meta = r.read_metadata()
        names = meta.get("tensor_names") or [f"tensor_{i}" for i in range(r.num_tensors)]
        dts = meta.get("tensor_dtypes")
        for i, name in enumerate(names[: r.num_tensors]):
            shape, code, nbytes = r.tensor_info(i)
            dt = getattr(torch, dts[i]) if dts else CODE_DTYPES.get(code, torch.float32)
            raw = r.read_tensor(i)
            t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt) if nbytes else torch.empty(0, dtype=dt)
            out[name] = t.view(*shape).to(device) if shape else t.reshape(()).to(device)
    return out, meta


class AsyncSaver:
    """Background writer with bounded staging (two checkpoints in flight by default): ``submit`` copies the tensors
    into host staging and returns; the write happens on the saver thread (kernel/distributed/checkpoint.c:52-301 of
    the reference describes the same double-buffered design but synchronises before writing)."""

    def __init__(self, max_pending: int = 2):
        self._h = _lib().sx_ckpt_saver_create(max_pending)

    def submit(self, path: str, parts, meta: dict):
        n, shapes, ndims, dtypes, ptrs, nbytes, strides, keep = _pack_args(parts)
        m = json.dumps(meta).encode("utf-8") if meta else None
        rc = _lib().sx_ckpt_saver_submit(self._h, path.encode(), n, shapes, ndims, dtypes, ptrs, nbytes, m)
        if rc != 0:
            raise IOError(f"queueing {path} failed ({rc})")

    def wait(self) -> int:
        return _lib().sx_ckpt_saver_wait(self._h)

    def close(self):
        if self._h:
            _lib().sx_ckpt_saver_destroy(self._h)
            self._h = None


# ---- the C trainer's raw checkpoint (kernel/train/trainer.c:269-353): u32 magic 0x41524958, u32 version 2, u64 step,
# u64 tensor count, then per tensor u32 ndim, u64 shape[ndim], u64 element count, fp32 data. Unnamed, in parameter order.
RAW_MAGIC, RAW_VERSION = 0x41524958, 2


def save_raw_trainer_checkpoint(path: str, step: int, tensors) -> None:
    """`tensors`: parameters in model order (a list, or the values of a state dict); stored as fp32."""
    import struct
    vals = list(tensors.values()) if isinstance(tensors, dict) else list(tensors)
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", RAW_MAGIC, RAW_VERSION, int(step), len(vals)))
        for t in vals:
            t = t.detach().float().cpu().contiguous()
            if t.dim() > 8:
                raise ValueError("the raw trainer format holds at most 8 dimensions")
            f.write(struct.pack("<I", t.dim()) + struct.pack(f"<{t.dim()}Q", *t.shape) + struct.pack("<Q", t.numel()))
            f.write(t.numpy().tobytes())


def load_raw_trainer_checkpoint(path: str):
    """-> (step, [fp32 tensors in file order]). Version 1 files carry the step only."""
    import struct
    import numpy as np
    data = open(path, "rb").read()
    if len(data) < 16 or struct.unpack_from("<I", data, 0)[0] != RAW_MAGIC:
        raise ValueError("not a raw trainer checkpoint")
    version, step = struct.unpack_from("<IQ", data, 4)
    if version not in (1, 2):
        raise ValueError(f"unsupported raw trainer checkpoint version {version}")
    if version == 1:
        return step, []
    if len(data) < 24:
        raise ValueError("raw trainer checkpoint truncated")
    (count,) = struct.unpack_from("<Q", data, 16)
    pos, out = 24, []
    if count > len(data):
        raise ValueError("tensor count larger than the file")
    for _ in range(count):
        if pos + 4 > len(data):
            raise ValueError("raw trainer checkpoint truncated")
        (nd,) = struct.unpack_from("<I", data, pos)
        pos += 4
        if nd > 8 or pos + 8 * nd + 8 > len(data):
            raise ValueError("bad tensor record")
        shape = struct.unpack_from(f"<{nd}Q", data, pos)
        pos += 8 * nd
        (n,) = struct.unpack_from("<Q", data, pos)
        pos += 8
        want = 1
        for d in shape:
            want *= d
        if n != want or pos + 4 * n > len(data):
            raise ValueError("tensor data does not match its shape or the file length")
        out.append(torch.from_numpy(np.frombuffer(data, dtype="<f4", count=n, offset=pos).reshape(shape).copy()))
        pos += 4 * n
    return step, out
