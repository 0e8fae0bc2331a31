"""Weight file formats beside `.sneppx`: safetensors (header JSON + raw tensors; fs/format/safetensors.c of the
reference), NumPy .npy/.npz, and the hub's native big-endian container (model_hub/converters/sneppx_format.py:10-142:
magic b"SNEPPX0001", u32 version, u32 meta size, JSON meta, u32 n, then per tensor name / dims / dtype code / bytes)."""
from __future__ import annotations

import json
import struct
from typing import Dict, Tuple

import numpy as np
import torch

_ST_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
              "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "I8": torch.int8, "BOOL": torch.bool,
              "F8_E4M3": torch.float8_e4m3fn}
_ST_NAMES = {v: k for k, v in _ST_DTYPES.items()}


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None):
    header, blobs, off = {}, [], 0
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def load_safetensors(path: str, device="cpu") -> Tuple[Dict[str, torch.Tensor], Dict[str, str]]:
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    meta = header.pop("__metadata__", {})
    out = {}
    for name, info in header.items():
        s, e = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        t = torch.frombuffer(bytearray(data[s:e]), dtype=torch.uint8).view(dt) if e > s else torch.empty(0, dtype=dt)
        out[name] = t.view(*info["shape"]).to(device)
    return out, meta


HUB_MAGIC = b"SNEPPX0001"
_HUB_CODES = {torch.float32: 1, torch.float16: 2, torch.int32: 3, torch.int64: 4, torch.uint8: 5}
_HUB_DTYPES = {v: k for k, v in _HUB_CODES.items()}


def save_hub_container(path: str, tensors: Dict[str, torch.Tensor], meta: dict = None):
    meta = dict(meta or {})
    meta["_tensors"] = list(tensors)
    mj = json.dumps(meta).encode()
    with open(path, "wb") as f:
        f.write(HUB_MAGIC)
        f.write(struct.pack(">II", 1, len(mj)))
        f.write(mj)
        f.write(struct.pack(">I", len(tensors)))
        for name, t in tensors.items():
            t = t.detach().cpu().contiguous()
            if t.dtype not in _HUB_CODES:
                t = t.float()
            nb = name.encode()
            raw = t.numpy().tobytes()
            f.write(struct.pack(">I", len(nb)) + nb + struct.pack(">I", t.dim()))
            f.write(struct.pack(f">{t.dim()}I", *t.shape) if t.dim() else b"")
            f.write(struct.pack(">IQ", _HUB_CODES[t.dtype], len(raw)))
            f.write(raw)


def load_hub_container(path: str):
    with open(path, "rb") as f:
        if f.read(10) != HUB_MAGIC:
            raise ValueError("not a hub container")
        _, msz = struct.unpack(">II", f.read(8))
        meta = json.loads(f.read(msz))
        n = struct.unpack(">I", f.read(4))[0]
        out = {}
        for _ in range(n):
            ln = struct.unpack(">I", f.read(4))[0]
            name = f.read(ln).decode()
            nd = struct.unpack(">I", f.read(4))[0]
            dims = struct.unpack(f">{nd}I", f.read(4 * nd)) if nd else ()
            code, nbytes = struct.unpack(">IQ", f.read(12))
            dt = _HUB_DTYPES[code]
            out[name] = torch.frombuffer(bytearray(f.read(nbytes)), dtype=dt).view(*dims) if nbytes else torch.empty(dims, dtype=dt)
    return out, meta


def save_npz(path, tensors):
    np.savez(path, **{k: v.detach().float().cpu().numpy() for k, v in tensors.items()})


def load_npz(path):
    with np.load(path) as z:
        return {k: torch.from_numpy(z[k]) for k in z.files}


def save_npy(path, tensor):
    np.save(path, tensor.detach().cpu().numpy() if tensor.dtype != torch.bfloat16 else tensor.detach().float().cpu().numpy())


def load_npy(path):
    return torch.from_numpy(np.load(path, allow_pickle=False))


def save_pth(path, state_dict: Dict[str, torch.Tensor]):
    """PyTorch ``.pth`` state dict (zip archive with a pickle of tensor stubs; fs/format/pth_format.c reads the same
    subset: tensors only, no arbitrary objects)."""
    torch.save({k: v.detach().cpu() for k, v in state_dict.items()}, path)


def load_pth(path, device="cpu") -> Dict[str, torch.Tensor]:
    """Loads a ``.pth`` / ``.pt`` state dict with the restricted unpickler (tensors and plain containers only); a
    checkpoint that wraps the weights under ``state_dict`` / ``model`` is unwrapped."""
    obj = torch.load(path, map_location=device, weights_only=True)
    for key in ("state_dict", "model", "model_state_dict"):
        if isinstance(obj, dict) and key in obj and isinstance(obj[key], dict):
            obj = obj[key]
    if not isinstance(obj, dict) or not all(torch.is_tensor(v) for v in obj.values()):
        raise ValueError(f"{path} does not hold a tensor state dict")
    return obj


def load_any(path, device="cpu") -> Dict[str, torch.Tensor]:
    """Dispatch on the file extension: .safetensors, .sneppx, .pth / .pt / .bin, .npz."""
    p = path.lower()
    if p.endswith(".safetensors"):
        return load_safetensors(path, device)[0]
    if p.endswith(".sneppx"):
        from ..checkpoint.sneppx_format import load_tensors
        return load_tensors(path)[0]
    if p.endswith((".pth", ".pt", ".bin")):
        return load_pth(path, device)
    if p.endswith(".npz"):
        return load_npz(path)
    raise ValueError(f"unknown weight file type: {path}")
