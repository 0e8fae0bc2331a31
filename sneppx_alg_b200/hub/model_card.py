"""Model cards and weight collections of the model zoo.

``ModelCard`` mirrors the record of the reference (``include/neural_core/model_zoo/model_card.h:23-77``: identity,
architecture, training, metrics, usage, tags, files; JSON round trip, validation) and adds a Markdown rendering and
``from_model``. ``WeightCollection`` is the reference's named-tensor container (``model_zoo/weights.h``: add / get /
remove / names, dtype conversion, int8 / int4 quantisation, load / save by format, memory-mapped loading); its GGUF
loader, a stub in the reference (``weights.c:278-281``), is implemented here for F32 / F16 / BF16 / Q8_0 tensors.
"""
from __future__ import annotations

import json
import struct
from dataclasses import asdict, dataclass, field, fields
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from . import formats


@dataclass
class ModelCard:
    name: str = ""
    version: str = ""
    description: str = ""
    author: str = ""
    license: str = ""
    repository: str = ""
    homepage: str = ""
    architecture: str = ""
    model_type: str = ""          # "causal-lm", "seq2seq", "vision", ...
    framework: str = "sneppx"
    num_parameters: int = 0
    num_layers: int = 0
    hidden_size: int = 0
    vocab_size: int = 0
    max_seq_len: int = 0
    training_data: str = ""
    training_procedure: str = ""
    optimizer: str = ""
    learning_rate: float = 0.0
    batch_size: int = 0
    num_epochs: int = 0
    precision: str = ""
    perplexity: float = 0.0
    accuracy: float = 0.0
    f1_score: float = 0.0
    latency_ms: float = 0.0
    throughput: float = 0.0
    intended_use: str = ""
    limitations: str = ""
    ethical_considerations: str = ""
    citation: str = ""
    tags: List[str] = field(default_factory=list)
    config_path: str = ""
    weights_path: str = ""
    tokenizer_path: str = ""

    def add_tag(self, tag: str):
        if tag not in self.tags:
            self.tags.append(tag)

    def validate(self) -> Tuple[bool, List[str]]:
        errors = []
        for f in ("name", "version", "architecture"):
            if not getattr(self, f):
                errors.append(f"{f} is required")
        for f in ("num_parameters", "num_layers", "hidden_size", "vocab_size", "max_seq_len", "batch_size", "num_epochs"):
            if getattr(self, f) < 0:
                errors.append(f"{f} must not be negative")
        if self.precision and self.precision not in ("fp32", "fp16", "bf16", "fp8", "int8", "int4", "mixed"):
            errors.append(f"unknown precision {self.precision!r}")
        if not 0.0 <= self.accuracy <= 1.0 or not 0.0 <= self.f1_score <= 1.0:
            errors.append("accuracy and f1_score are fractions in [0, 1]")
        return not errors, errors

    def to_json(self, pretty: bool = True) -> str:
        return json.dumps(asdict(self), indent=2 if pretty else None, sort_keys=True)

    @classmethod
    def from_json(cls, text: str) -> "ModelCard":
        raw = json.loads(text)
        if not isinstance(raw, dict):
            raise ValueError("a model card is a JSON object")
        known = {f.name: f for f in fields(cls)}
        card = cls()
        for k, v in raw.items():
            if k not in known:
                continue                                   # cards written by newer versions may carry more fields
            want = type(getattr(card, k))
            if want is float and isinstance(v, int):
                v = float(v)
            if not isinstance(v, want):
                raise ValueError(f"field {k} must be {want.__name__}")
            setattr(card, k, v)
        return card

    def save(self, path: str):
        with open(path, "w") as f:
            f.write(self.to_json())

    @classmethod
    def load(cls, path: str) -> "ModelCard":
        return cls.from_json(open(path).read())

    @classmethod
    def from_model(cls, model: torch.nn.Module, name: str, version: str = "1.0.0", **extra) -> "ModelCard":
        cfg = getattr(model, "config", None)
        g = lambda *names: next((int(getattr(cfg, n)) for n in names if cfg is not None and getattr(cfg, n, None)), 0)  # noqa: E731
        p = next(model.parameters(), None)
        prec = {torch.float32: "fp32", torch.float16: "fp16", torch.bfloat16: "bf16"}.get(p.dtype if p is not None else None, "")
        return cls(name=name, version=version, architecture=type(model).__name__, num_parameters=sum(q.numel() for q in model.parameters()),
                   num_layers=g("num_hidden_layers", "n_layer", "num_layers"), hidden_size=g("hidden_size", "d_model"),
                   vocab_size=g("vocab_size"), max_seq_len=g("max_position_embeddings", "max_seq_len"), precision=prec, **extra)

    def to_markdown(self) -> str:
        lines = [f"# {self.name} {self.version}".rstrip(), "", self.description, ""]
        rows = [("Architecture", self.architecture), ("Type", self.model_type), ("Parameters", f"{self.num_parameters:,}" if self.num_parameters else ""),
                ("Layers", self.num_layers or ""), ("Hidden size", self.hidden_size or ""), ("Vocabulary", self.vocab_size or ""),
                ("Context", self.max_seq_len or ""), ("Precision", self.precision), ("License", self.license), ("Author", self.author)]
        lines += ["| | |", "|---|---|"] + [f"| {k} | {v} |" for k, v in rows if v != ""]
        for title, text in (("Intended use", self.intended_use), ("Limitations", self.limitations),
                            ("Ethical considerations", self.ethical_considerations), ("Training data", self.training_data),
                            ("Citation", self.citation)):
            if text:
                lines += ["", f"## {title}", "", text]
        if self.tags:
            lines += ["", "Tags: " + ", ".join(self.tags)]
        return "\n".join(lines) + "\n"


# ------------------------------------------------------------------------------------------------- GGUF
_GGUF_MAGIC = b"GGUF"
_GGML_F32, _GGML_F16, _GGML_Q8_0, _GGML_BF16 = 0, 1, 8, 30
_KV_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class _Reader:
    def __init__(self, data: bytes):
        self.d, self.p = data, 0

    def take(self, fmt: str):
        n = struct.calcsize(fmt)
        if self.p + n > len(self.d):
            raise ValueError("GGUF file truncated")
        (v,) = struct.unpack_from(fmt, self.d, self.p)
        self.p += n
        return v

    def string(self) -> str:
        n = self.take("<Q")
        if self.p + n > len(self.d):
            raise ValueError("GGUF string runs past the end of the file")
        s = self.d[self.p:self.p + n].decode("utf-8", "replace")
        self.p += n
        return s

    def value(self, t: int, depth: int = 0):
        if t in _KV_FMT:
            return self.take(_KV_FMT[t])
        if t == 8:
            return self.string()
        if t == 9 and depth < 4:
            et, n = self.take("<I"), self.take("<Q")
            if n > len(self.d):
                raise ValueError("GGUF array longer than the file")
            return [self.value(et, depth + 1) for _ in range(n)]
        raise ValueError(f"unknown GGUF value type {t}")


def load_gguf(path: str) -> Tuple[Dict[str, torch.Tensor], dict]:
    """(tensors, metadata) of a GGUF v2 / v3 file. F32, F16 and BF16 tensors load as they are; Q8_0 (blocks of 32 int8
    with one fp16 scale) is expanded to fp32. Shapes come back outermost-first (GGUF stores the innermost first)."""
    data = open(path, "rb").read()
    r = _Reader(data)
    if data[:4] != _GGUF_MAGIC:
        raise ValueError("not a GGUF file")
    r.p = 4
    version, n_tensors, n_kv = r.take("<I"), r.take("<Q"), r.take("<Q")
    if version not in (2, 3) or n_tensors > 1 << 20 or n_kv > 1 << 20:
        raise ValueError("unsupported GGUF header")
    meta = {}
    for _ in range(n_kv):
        k = r.string()
        meta[k] = r.value(r.take("<I"))
    infos = []
    for _ in range(n_tensors):
        name, nd = r.string(), r.take("<I")
        if nd > 8:
            raise ValueError("tensor with too many dimensions")
        dims = [r.take("<Q") for _ in range(nd)]
        infos.append((name, dims, r.take("<I"), r.take("<Q")))
    align = int(meta.get("general.alignment", 32)) or 32
    base = (r.p + align - 1) // align * align
    out = {}
    for name, dims, t, off in infos:
        n = int(np.prod(dims)) if dims else 1
        shape = tuple(reversed(dims))
        nbytes = {_GGML_F32: 4 * n, _GGML_F16: 2 * n, _GGML_BF16: 2 * n, _GGML_Q8_0: n // 32 * 34}.get(t)
        if nbytes is None:
            raise ValueError(f"tensor {name}: GGML type {t} is not supported")
        if base + off + nbytes > len(data):
            raise ValueError(f"tensor {name} runs past the end of the file")
        raw = np.frombuffer(data, dtype=np.uint8, count=nbytes, offset=base + off)
        if t == _GGML_F32:
            out[name] = torch.from_numpy(raw.view("<f4").reshape(shape).copy())
        elif t == _GGML_F16:
            out[name] = torch.from_numpy(raw.view("<f2").reshape(shape).copy())
        elif t == _GGML_BF16:
            out[name] = torch.from_numpy(raw.view("<i2").reshape(shape).copy()).view(torch.bfloat16)
        else:
            if n % 32:
                raise ValueError(f"tensor {name}: Q8_0 needs a multiple of 32 elements")
            blocks = raw.reshape(-1, 34)
            scale = blocks[:, :2].copy().view("<f2").astype(np.float32)
            q = blocks[:, 2:].view(np.int8).astype(np.float32)
            out[name] = torch.from_numpy((q * scale).reshape(shape))
    return out, meta


def save_gguf(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[dict] = None, q8_0: bool = False):
    """Writes GGUF v3. Metadata values may be str, bool, int, float or flat lists of those. With `q8_0`, 2-D float
    tensors whose row length is a multiple of 32 are stored as Q8_0."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    def val(v) -> bytes:
        if isinstance(v, bool):
            return struct.pack("<I?", 7, v)
        if isinstance(v, int):
            return struct.pack("<Iq", 11, v) if v < 0 else struct.pack("<IQ", 10, v)
        if isinstance(v, float):
            return struct.pack("<Id", 12, v)
        if isinstance(v, str):
            return struct.pack("<I", 8) + s(v)
        if isinstance(v, (list, tuple)):
            items = [val(x) for x in v] or [val("")]
            et = items[0][:4]
            if any(i[:4] != et for i in items):
                raise ValueError("GGUF arrays hold one value type")
            return struct.pack("<I", 9) + et + struct.pack("<Q", len(v)) + b"".join(i[4:] for i in items[:len(v)])
        raise TypeError(f"cannot store {type(v).__name__} in GGUF metadata")

    meta = dict(metadata or {})
    meta.setdefault("general.alignment", 32)
    align = int(meta["general.alignment"])
    head = _GGUF_MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += s(k) + (struct.pack("<II", 4, v) if k == "general.alignment" else val(v))
    blobs, infos, off = [], b"", 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if q8_0 and t.dim() == 2 and t.is_floating_point() and t.shape[-1] % 32 == 0:
            g = t.float().reshape(-1, 32)
            scale = (g.abs().amax(1, keepdim=True) / 127.0).half()
            q = torch.round(g / scale.float().clamp_min(1e-12)).clamp(-127, 127).to(torch.int8)
            blob = np.concatenate([scale.numpy().view(np.uint8).reshape(-1, 2), q.numpy().view(np.uint8)], axis=1).tobytes()
            code = _GGML_Q8_0
        elif t.dtype == torch.bfloat16:
            blob, code = t.view(torch.int16).numpy().tobytes(), _GGML_BF16
        elif t.dtype == torch.float16:
            blob, code = t.numpy().tobytes(), _GGML_F16
        else:
            blob, code = t.float().numpy().tobytes(), _GGML_F32
        infos += s(name) + struct.pack("<I", t.dim()) + b"".join(struct.pack("<Q", d) for d in reversed(t.shape)) + struct.pack("<IQ", code, off)
        pad = (-len(blob)) % align
        blobs.append(blob + b"\0" * pad)
        off += len(blob) + pad
    body = head + infos
    with open(path, "wb") as f:
        f.write(body + b"\0" * ((-len(body)) % align))
        for b in blobs:
            f.write(b)


# ------------------------------------------------------------------------------------------------- weights
_DTYPES = {"fp32": torch.float32, "float32": torch.float32, "fp16": torch.float16, "float16": torch.float16,
           "bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp64": torch.float64, "float64": torch.float64}
_EXT_FORMAT = {".safetensors": "safetensors", ".gguf": "gguf", ".npz": "npz", ".pth": "pth", ".pt": "pth", ".sxh5": "sxh5"}


def dtype_size(name: str) -> int:
    if name in ("int8", "uint8", "fp8"):
        return 1
    if name in _DTYPES:
        return torch.empty((), dtype=_DTYPES[name]).element_size()
    raise ValueError(f"unknown dtype {name!r}")


class WeightCollection:
    """Named tensors with per-tensor quantisation state. Quantised entries keep (codes, scale) and expand on ``get``."""

    def __init__(self):
        self.tensors: Dict[str, torch.Tensor] = {}
        self.quant: Dict[str, dict] = {}
        self.metadata: dict = {}

    # ---- container
    def add(self, name: str, tensor: torch.Tensor):
        self.tensors[name] = tensor
        self.quant.pop(name, None)

    def get(self, name: str, dequantize: bool = True) -> torch.Tensor:
        from ..quant import algorithms as qa
        t = self.tensors[name]
        q = self.quant.get(name)
        if q is None or not dequantize:
            return t
        if q["kind"] == "int8":
            return qa.dequantize_int8(t, q["scale"]).to(q["dtype"])
        return qa.dequantize_int4_packed(t, q["scale"], q["group"]).reshape(q["shape"]).to(q["dtype"])

    def remove(self, name: str) -> bool:
        self.quant.pop(name, None)
        return self.tensors.pop(name, None) is not None

    def names(self) -> List[str]:
        return list(self.tensors)

    def __len__(self):
        return len(self.tensors)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values()) + \
            sum(q["scale"].numel() * 4 for q in self.quant.values())

    # ---- conversions
    def convert_dtype(self, target: str, names: Optional[List[str]] = None):
        dt = _DTYPES[target]
        for n in names or self.names():
            if n not in self.quant and self.tensors[n].is_floating_point():
                self.tensors[n] = self.tensors[n].to(dt)

    def quantize_int8(self, name: str):
        """Per-output-channel symmetric int8 for matrices, per-tensor for everything else."""
        from ..quant import algorithms as qa
        t = self.get(name)
        mode = qa.QuantMode.INT8_PER_CHANNEL if t.dim() >= 2 else qa.QuantMode.INT8_SYMMETRIC
        q, scale, _ = qa.quantize_int8(t, mode)
        self.tensors[name], self.quant[name] = q, {"kind": "int8", "scale": scale.float(), "dtype": t.dtype}

    def quantize_int4(self, name: str, group: int = 128):
        from ..quant import algorithms as qa
        t = self.get(name)
        if t.shape[-1] % group:
            raise ValueError(f"{name}: last dimension {t.shape[-1]} is not a multiple of the group size {group}")
        packed, scale = qa.quantize_int4_packed(t, group)
        self.tensors[name] = packed
        self.quant[name] = {"kind": "int4", "scale": scale.float(), "group": group, "shape": tuple(t.shape), "dtype": t.dtype}

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {n: self.get(n) for n in self.names()}

    # ---- files
    @staticmethod
    def format_of(path: str) -> str:
        import os
        ext = os.path.splitext(path)[1].lower()
        if ext not in _EXT_FORMAT:
            raise ValueError(f"cannot tell the weight format of {path!r}")
        return _EXT_FORMAT[ext]

    @classmethod
    def load(cls, path: str, fmt: Optional[str] = None, mmap: bool = False) -> "WeightCollection":
        """`mmap`: safetensors and the hierarchical store are mapped, so tensors are paged in when first touched."""
        wc, fmt = cls(), fmt or cls.format_of(path)
        if fmt == "gguf":
            tensors, wc.metadata = load_gguf(path)
        elif fmt == "safetensors":
            if mmap:
                tensors, wc.metadata = _mmap_safetensors(path)
            else:
                tensors, wc.metadata = formats.load_safetensors(path)
        elif fmt == "npz":
            tensors = formats.load_npz(path)
        elif fmt == "pth":
            tensors = formats.load_pth(path)
        elif fmt == "sxh5":
            with formats.HierarchicalFile(path, "r") as f:
                tensors = f.read_state_dict("/")
        else:
            raise ValueError(f"unknown weight format {fmt!r}")
        for k, v in tensors.items():
            wc.tensors[k] = v if isinstance(v, torch.Tensor) else torch.as_tensor(np.asarray(v))
        return wc

    def save(self, path: str, fmt: Optional[str] = None):
        fmt = fmt or self.format_of(path)
        sd = {k: v.contiguous() for k, v in self.state_dict().items()}
        if fmt == "gguf":
            save_gguf(path, sd, {k: v for k, v in self.metadata.items() if isinstance(v, (str, int, float, bool, list))})
        elif fmt == "safetensors":
            formats.save_safetensors(path, sd, {k: str(v) for k, v in self.metadata.items()})
        elif fmt == "npz":
            formats.save_npz(path, sd)
        elif fmt == "pth":
            formats.save_pth(path, sd)
        elif fmt == "sxh5":
            with formats.HierarchicalFile(path, "w") as f:
                f.write_state_dict(sd)
        else:
            raise ValueError(f"unknown weight format {fmt!r}")


def _mmap_safetensors(path: str):
    """Zero-copy view of a safetensors file: header parsed, every tensor a slice of one read-only memory map."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        size = f.seek(0, 2)
        if n > size - 8:
            raise ValueError("safetensors header longer than the file")
        f.seek(8)
        header = json.loads(f.read(n))
    meta = header.pop("__metadata__", {})
    mm = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + n) if size > 8 + n else np.zeros(0, dtype=np.uint8)
    kinds = {"F32": ("<f4", None), "F16": ("<f2", None), "BF16": ("<i2", torch.bfloat16), "F64": ("<f8", None), "I64": ("<i8", None),
             "I32": ("<i4", None), "I16": ("<i2", None), "I8": ("i1", None), "U8": ("u1", None), "BOOL": ("?", None)}
    out = {}
    for name, e in header.items():
        if e["dtype"] not in kinds:
            raise ValueError(f"{name}: dtype {e['dtype']} is not supported")
        lo, hi = e["data_offsets"]
        if not 0 <= lo <= hi <= mm.size:
            raise ValueError(f"{name}: data offsets outside the file")
        np_dt, view = kinds[e["dtype"]]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                # torch warns that the mapped array is read-only
            t = torch.from_numpy(mm[lo:hi].view(np_dt).reshape(e["shape"]))
        out[name] = t.view(view) if view is not None else t
    return out, meta
