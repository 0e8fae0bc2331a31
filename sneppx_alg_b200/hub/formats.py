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
    """Dispatch on the file extension: .safetensors, .sneppx, .pth / .pt / .bin, .npz, .gguf, .sxh5."""
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
    if p.endswith(".gguf"):
        from .model_card import load_gguf
        return load_gguf(path)[0]
    if p.endswith(".sxh5"):
        with HierarchicalFile(path, "r") as f:
            return f.read_state_dict("/")
    raise ValueError(f"unknown weight file type: {path}")


class HierarchicalFile:
    """Single-file hierarchical store: groups, n-dimensional datasets and attributes addressed by ``/a/b/c`` paths
    (the API of the reference's HDF5-like format, ``fs/format/hdf5_format.h:31-115``: open / create_group /
    dataset_exists / read_dataset / write_dataset / read_attribute / write_attribute / list_children; its body keeps
    the tree in memory only).

    Layout: ``SXH5`` magic, version, the byte offset of the index (u64), then dataset payloads appended on 64-byte
    boundaries, then a JSON index {path: {"kind", "dtype", "shape", "offset", "nbytes", "attrs"}}. Appending rewrites
    only the index; replaced datasets leave their old payload behind until ``repack``. Datasets are read through a
    memory map, so opening a file of any size costs the index only."""

    MAGIC = b"SXH5"

    def __init__(self, path: str, mode: str = "r"):
        import os
        if mode not in ("r", "w", "a"):
            raise ValueError("mode must be 'r', 'w' or 'a'")
        self.path, self.mode, self._dirty = path, mode, False
        if mode == "w" or (mode == "a" and not os.path.exists(path)):
            self.index = {"/": {"kind": "group", "attrs": {}}}
            with open(path, "wb") as f:
                f.write(self.MAGIC + struct.pack("<IQ", 1, 16))
            self._end = 16
            self._dirty = True
        else:
            with open(path, "rb") as f:
                head = f.read(16)
                if len(head) != 16 or head[:4] != self.MAGIC:
                    raise ValueError("not a hierarchical store file")
                _, off = struct.unpack("<IQ", head[4:])
                size = f.seek(0, 2)
                if off < 16 or off > size:
                    raise ValueError("index offset outside the file")
                f.seek(off)
                try:
                    self.index = json.loads(f.read().decode())
                except Exception as e:
                    raise ValueError("corrupt index") from e
            for p, e in self.index.items():
                if e.get("kind") == "dataset" and e["offset"] + e["nbytes"] > off:
                    raise ValueError(f"dataset {p} extends past the data region")
            self._end = off

    # ---- tree
    @staticmethod
    def _norm(path: str) -> str:
        parts = [p for p in path.split("/") if p]
        return "/" + "/".join(parts)

    def create_group(self, path: str):
        self._writable()
        parts = [p for p in path.split("/") if p]
        for i in range(1, len(parts) + 1):
            p = "/" + "/".join(parts[:i])
            e = self.index.setdefault(p, {"kind": "group", "attrs": {}})
            if e["kind"] != "group":
                raise ValueError(f"{p} is a dataset")
        self._dirty = True

    def exists(self, path: str) -> bool:
        return self._norm(path) in self.index

    def dataset_exists(self, path: str) -> bool:
        return self.index.get(self._norm(path), {}).get("kind") == "dataset"

    def list_children(self, path: str = "/"):
        base = self._norm(path).rstrip("/") + "/"
        return sorted({p[len(base):].split("/")[0] for p in self.index if p.startswith(base) and p != base and p != "/"})

    def _writable(self):
        if self.mode == "r":
            raise PermissionError("file opened read-only")

    # ---- datasets
    def write_dataset(self, path: str, data):
        self._writable()
        a = data.detach().cpu().numpy() if isinstance(data, torch.Tensor) and data.dtype != torch.bfloat16 else data
        bf16 = isinstance(a, torch.Tensor)
        if bf16:                                                       # bfloat16 has no NumPy dtype: store the bit pattern
            a = a.detach().cpu().view(torch.int16).numpy()
        a = np.ascontiguousarray(a)
        p = self._norm(path)
        if "/" in p[1:]:
            self.create_group(p.rsplit("/", 1)[0])
        if self.index.get(p, {}).get("kind") == "group":
            raise ValueError(f"{p} is a group")
        off = (self._end + 63) // 64 * 64
        with open(self.path, "r+b") as f:
            f.seek(off)
            f.write(a.tobytes())
        self.index[p] = {"kind": "dataset", "dtype": "bfloat16" if bf16 else a.dtype.str, "shape": list(a.shape), "offset": off,
                         "nbytes": a.nbytes, "attrs": self.index.get(p, {}).get("attrs", {})}
        self._end = off + a.nbytes
        self._dirty = True

    def read_dataset(self, path: str, as_tensor: bool = False):
        e = self.index.get(self._norm(path))
        if e is None or e["kind"] != "dataset":
            raise KeyError(path)
        self.flush()
        bf16 = e["dtype"] == "bfloat16"
        dt = np.dtype("<i2") if bf16 else np.dtype(e["dtype"])
        if e["nbytes"] == 0:
            a = np.zeros(e["shape"], dtype=dt)
        else:
            a = np.memmap(self.path, dtype=dt, mode="r", offset=e["offset"], shape=tuple(e["shape"]))
        if bf16:
            return torch.from_numpy(np.array(a)).view(torch.bfloat16)
        return torch.from_numpy(np.array(a)) if as_tensor else a

    # ---- attributes (JSON values, or bytes stored as hex)
    def write_attribute(self, path: str, name: str, value):
        self._writable()
        p = self._norm(path)
        if p not in self.index:
            self.create_group(p)
        self.index[p]["attrs"][name] = {"hex": value.hex()} if isinstance(value, (bytes, bytearray)) else {"json": value}
        self._dirty = True

    def read_attribute(self, path: str, name: str):
        v = self.index[self._norm(path)]["attrs"][name]
        return bytes.fromhex(v["hex"]) if "hex" in v else v["json"]

    # ---- whole-model helpers
    def write_state_dict(self, state: Dict[str, torch.Tensor], root: str = "/"):
        for k, v in state.items():
            self.write_dataset(self._norm(root) + "/" + k.replace(".", "/"), v)

    def read_state_dict(self, root: str = "/") -> Dict[str, torch.Tensor]:
        base = self._norm(root).rstrip("/") + "/"
        return {p[len(base):].replace("/", "."): self.read_dataset(p, as_tensor=True)
                for p, e in self.index.items() if e["kind"] == "dataset" and p.startswith(base)}

    def repack(self):
        """Rewrites the file without the payloads that replaced datasets left behind."""
        self._writable()
        import os
        live = {p: np.array(self.read_dataset(p)) if e["dtype"] != "bfloat16" else self.read_dataset(p)
                for p, e in self.index.items() if e["kind"] == "dataset"}
        tmp = HierarchicalFile(self.path + ".repack", "w")
        for p, e in self.index.items():
            if e["kind"] == "group":
                tmp.create_group(p)
        for p, a in live.items():
            tmp.write_dataset(p, a)
        for p, e in self.index.items():
            tmp.index[p]["attrs"] = e["attrs"]
        tmp._dirty = True
        tmp.close()
        os.replace(self.path + ".repack", self.path)
        self.index, self._end, self._dirty = tmp.index, tmp._end, False

    def flush(self):
        if self._dirty and self.mode != "r":
            blob = json.dumps(self.index).encode()
            with open(self.path, "r+b") as f:
                f.seek(self._end)
                f.write(blob)
                f.truncate()
                f.seek(4)
                f.write(struct.pack("<IQ", 1, self._end))
            self._dirty = False

    def close(self):
        self.flush()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
