"""Stand-alone ONNX toolkit (no onnx / onnxruntime dependency): protobuf wire codec, model parser / serialiser,
checker, shape inference, optimiser (constant folding + dead-code elimination), QDQ quantiser, NumPy executor and an
exporter for feed-forward torch modules. Same scope as the reference's ``onnx/`` package (onnx/*.py, 3.7 K lines) and
``onnx_export.py`` / ``onnx_check.py`` bindings."""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

# ----------------------------------------------------------------------------- protobuf wire format
def _varint(n: int) -> bytes:
    n &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = val = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _ld(num: int, data: bytes) -> bytes:
    return _field(num, 2, _varint(len(data)) + data)


def _vi(num: int, v: int) -> bytes:
    return _field(num, 0, _varint(v))


def parse_message(buf: bytes) -> List[Tuple[int, int, Any]]:
    """[(field number, wire type, value)] with length-delimited values left as bytes."""
    out, pos = [], 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        num, wire = key >> 3, key & 7
        if wire == 0:
            v, pos = _read_varint(buf, pos)
        elif wire == 1:
            v = buf[pos: pos + 8]
            pos += 8
        elif wire == 2:
            n, pos = _read_varint(buf, pos)
            v = buf[pos: pos + n]
            pos += n
        elif wire == 5:
            v = buf[pos: pos + 4]
            pos += 4
        else:
            raise ValueError(f"unsupported wire type {wire}")
        out.append((num, wire, v))
    return out


# ----------------------------------------------------------------------------- model objects
DT_FLOAT, DT_UINT8, DT_INT8, DT_INT32, DT_INT64, DT_FLOAT16, DT_DOUBLE, DT_BOOL = 1, 2, 3, 6, 7, 10, 11, 9
_NP = {DT_FLOAT: np.float32, DT_UINT8: np.uint8, DT_INT8: np.int8, DT_INT32: np.int32, DT_INT64: np.int64,
       DT_FLOAT16: np.float16, DT_DOUBLE: np.float64, DT_BOOL: np.bool_}
_DT = {np.dtype(v): k for k, v in _NP.items()}


@dataclass
class Tensor:
    name: str
    data: np.ndarray
    external: Optional[Dict[str, str]] = None     # {"location", "offset", "length"} when the bytes live in a side file

    def serialize(self, external: Optional[Dict[str, str]] = None) -> bytes:
        a = np.ascontiguousarray(self.data)
        out = b"".join(_vi(1, int(d)) for d in a.shape) + _vi(2, _DT[a.dtype]) + _ld(8, self.name.encode())
        if external is None:
            return out + _ld(9, a.tobytes())
        # TensorProto.external_data (field 13, key / value entries) + data_location = EXTERNAL (field 14)
        for k in ("location", "offset", "length"):
            out += _ld(13, _ld(1, k.encode()) + _ld(2, str(external[k]).encode()))
        return out + _vi(14, 1)

    @classmethod
    def parse(cls, buf: bytes) -> "Tensor":
        dims, dt, name, raw, floats, ints = [], DT_FLOAT, "", None, [], []
        ext, location = {}, 0
        for num, wire, v in parse_message(buf):
            if num == 13:
                kv = {n_: x for n_, _, x in parse_message(v)}
                ext[kv.get(1, b"").decode()] = kv.get(2, b"").decode()
                continue
            if num == 14:
                location = v
                continue
            if num == 1:
                dims.append(v) if wire == 0 else dims.extend(_unpack_varints(v))
            elif num == 2:
                dt = v
            elif num == 8:
                name = v.decode()
            elif num == 9:
                raw = v
            elif num == 4:
                floats.extend(struct.unpack(f"<{len(v) // 4}f", v) if wire == 2 else struct.unpack("<f", v))
            elif num == 7:
                ints.extend(_unpack_varints(v) if wire == 2 else [v])
        if location == 1:        # bytes are in a side file: placeholder of the right shape until they are loaded
            if "location" not in ext:
                raise ValueError(f"tensor {name!r} is marked external but names no file")
            return cls(name, np.zeros(dims, dtype=_NP[dt]), ext)
        if raw is not None:
            arr = np.frombuffer(raw, dtype=_NP[dt]).reshape(dims)
        elif floats:
            arr = np.array(floats, dtype=np.float32).reshape(dims)
        else:
            arr = np.array([_signed(i) for i in ints], dtype=_NP.get(dt, np.int64)).reshape(dims)
        return cls(name, arr.copy())


def _unpack_varints(buf: bytes) -> List[int]:
    out, pos = [], 0
    while pos < len(buf):
        v, pos = _read_varint(buf, pos)
        out.append(v)
    return out


def _signed(v: int) -> int:
    return v - (1 << 64) if v >= 1 << 63 else v


@dataclass
class Node:
    op_type: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)
    name: str = ""

    def serialize(self) -> bytes:
        out = b"".join(_ld(1, i.encode()) for i in self.inputs) + b"".join(_ld(2, o.encode()) for o in self.outputs)
        out += _ld(3, self.name.encode()) + _ld(4, self.op_type.encode())
        for k, v in self.attrs.items():
            a = _ld(1, k.encode())
            if isinstance(v, float):
                a += _field(2, 5, struct.pack("<f", v)) + _vi(20, 1)
            elif isinstance(v, (int, np.integer)):
                a += _vi(3, int(v)) + _vi(20, 2)
            elif isinstance(v, str):
                a += _ld(4, v.encode()) + _vi(20, 3)
            elif isinstance(v, np.ndarray):
                a += _ld(5, Tensor("", v).serialize()) + _vi(20, 4)
            elif isinstance(v, (list, tuple)) and all(isinstance(x, (int, np.integer)) for x in v):
                a += b"".join(_vi(8, int(x)) for x in v) + _vi(20, 7)
            elif isinstance(v, (list, tuple)):
                a += b"".join(_field(7, 5, struct.pack("<f", float(x))) for x in v) + _vi(20, 6)
            out += _ld(5, a)
        return out

    @classmethod
    def parse(cls, buf: bytes) -> "Node":
        n = cls("", [], [])
        for num, wire, v in parse_message(buf):
            if num == 1:
                n.inputs.append(v.decode())
            elif num == 2:
                n.outputs.append(v.decode())
            elif num == 3:
                n.name = v.decode()
            elif num == 4:
                n.op_type = v.decode()
            elif num == 5:
                name, val, ints, floats = "", None, [], []
                for an, aw, av in parse_message(v):
                    if an == 1:
                        name = av.decode()
                    elif an == 2:
                        val = struct.unpack("<f", av)[0]
                    elif an == 3:
                        val = _signed(av)
                    elif an == 4:
                        val = av.decode()
                    elif an == 5:
                        val = Tensor.parse(av).data
                    elif an == 7:
                        floats.extend(struct.unpack(f"<{len(av) // 4}f", av) if aw == 2 else struct.unpack("<f", av))
                    elif an == 8:
                        ints.extend([_signed(i) for i in _unpack_varints(av)] if aw == 2 else [_signed(av)])
                n.attrs[name] = val if val is not None else (ints if ints else floats)
        return n


@dataclass
class ValueInfo:
    name: str
    dtype: int = DT_FLOAT
    shape: Tuple = ()

    def serialize(self) -> bytes:
        dims = b"".join(_ld(1, _ld(2, str(d).encode()) if isinstance(d, str) else _vi(1, int(d))) for d in self.shape)
        ttype = _vi(1, self.dtype) + _ld(2, dims)
        return _ld(1, self.name.encode()) + _ld(2, _ld(1, ttype))

    @classmethod
    def parse(cls, buf: bytes) -> "ValueInfo":
        vi = cls("")
        for num, _, v in parse_message(buf):
            if num == 1:
                vi.name = v.decode()
            elif num == 2:
                for tn, _, tv in parse_message(v):
                    if tn == 1:
                        shape = []
                        for fn, _, fv in parse_message(tv):
                            if fn == 1:
                                vi.dtype = fv
                            elif fn == 2:
                                for dn, _, dv in parse_message(fv):
                                    d = None
                                    for xn, xw, xv in parse_message(dv):
                                        d = xv if xn == 1 else xv.decode()
                                    shape.append(d)
                        vi.shape = tuple(shape)
        return vi


@dataclass
class Graph:
    nodes: List[Node] = field(default_factory=list)
    inputs: List[ValueInfo] = field(default_factory=list)
    outputs: List[ValueInfo] = field(default_factory=list)
    initializers: Dict[str, np.ndarray] = field(default_factory=dict)
    name: str = "graph"


@dataclass
class Model:
    graph: Graph
    ir_version: int = 8
    opset: int = 17
    producer: str = "sneppx"
    external: Dict[str, Dict[str, str]] = field(default_factory=dict)   # initializers whose bytes are in side files

    def serialize(self) -> bytes:
        g = self.graph
        gb = b"".join(_ld(1, n.serialize()) for n in g.nodes) + _ld(2, g.name.encode())
        gb += b"".join(_ld(5, Tensor(k, v).serialize(self.external.get(k))) for k, v in g.initializers.items())
        gb += b"".join(_ld(11, v.serialize()) for v in g.inputs) + b"".join(_ld(12, v.serialize()) for v in g.outputs)
        return _vi(1, self.ir_version) + _ld(2, self.producer.encode()) + _ld(7, gb) + _ld(8, _ld(1, b"") + _vi(2, self.opset))

    @classmethod
    def parse(cls, buf: bytes) -> "Model":
        """Decodes a serialized ModelProto; any structural problem (truncated field, wrong wire type, bad UTF-8, a
        tensor whose data does not match its dims) is reported as ``ValueError``."""
        try:
            return cls._parse(buf)
        except ValueError:
            raise
        except (AttributeError, TypeError, IndexError, KeyError, struct.error, OverflowError, MemoryError) as e:
            raise ValueError(f"malformed ONNX model: {type(e).__name__}: {e}") from None

    @classmethod
    def _parse(cls, buf: bytes) -> "Model":
        m = cls(Graph())
        for num, _, v in parse_message(buf):
            if num == 1:
                m.ir_version = v
            elif num == 2:
                m.producer = v.decode()
            elif num == 8:
                for on, _, ov in parse_message(v):
                    if on == 2:
                        m.opset = ov
            elif num == 7:
                for gn, _, gv in parse_message(v):
                    if gn == 1:
                        m.graph.nodes.append(Node.parse(gv))
                    elif gn == 2:
                        m.graph.name = gv.decode()
                    elif gn == 5:
                        t = Tensor.parse(gv)
                        m.graph.initializers[t.name] = t.data
                        if t.external is not None:
                            m.external[t.name] = t.external
                    elif gn == 11:
                        m.graph.inputs.append(ValueInfo.parse(gv))
                    elif gn == 12:
                        m.graph.outputs.append(ValueInfo.parse(gv))
        return m

    def save(self, path: str):
        with open(path, "wb") as f:
            f.write(self.serialize())

    @classmethod
    def load(cls, path: str) -> "Model":
        with open(path, "rb") as f:
            return cls.parse(f.read())


# ----------------------------------------------------------------------------- checker / shapes / executor
def check_model(m: Model) -> List[str]:
    errs, known = [], set(m.graph.initializers) | {i.name for i in m.graph.inputs}
    if not m.graph.nodes:
        errs.append("graph has no nodes")
    for n in m.graph.nodes:
        if n.op_type not in OPS:
            errs.append(f"unsupported op {n.op_type}")
        for i in n.inputs:
            if i and i not in known:
                errs.append(f"node {n.name or n.op_type}: input '{i}' used before definition")
        for o in n.outputs:
            if o in known:
                errs.append(f"value '{o}' defined twice")
            known.add(o)
    for o in m.graph.outputs:
        if o.name not in known:
            errs.append(f"graph output '{o.name}' is never produced")
    return errs


def _softmax(x, axis=-1):
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


def _gemm(a, b, c=None, alpha=1.0, beta=1.0, transA=0, transB=0):
    y = alpha * ((a.T if transA else a) @ (b.T if transB else b))
    return y + beta * c if c is not None else y


def _layernorm(x, w, b=None, axis=-1, epsilon=1e-5):
    mu = x.mean(axis=axis, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=axis, keepdims=True)
    y = (x - mu) / np.sqrt(var + epsilon) * w
    return y + b if b is not None else y


OPS = {
    "MatMul": lambda a, i: i[0] @ i[1], "Gemm": lambda a, i: _gemm(*i, **{k: a[k] for k in ("alpha", "beta", "transA", "transB") if k in a}),
    "Add": lambda a, i: i[0] + i[1], "Sub": lambda a, i: i[0] - i[1], "Mul": lambda a, i: i[0] * i[1], "Div": lambda a, i: i[0] / i[1],
    "Relu": lambda a, i: np.maximum(i[0], 0), "Sigmoid": lambda a, i: 1 / (1 + np.exp(-i[0])), "Tanh": lambda a, i: np.tanh(i[0]),
    "Gelu": lambda a, i: 0.5 * i[0] * (1 + np.tanh(0.7978845608 * (i[0] + 0.044715 * i[0] ** 3))),
    "Softmax": lambda a, i: _softmax(i[0], a.get("axis", -1)), "Identity": lambda a, i: i[0],
    "LayerNormalization": lambda a, i: _layernorm(*i, axis=a.get("axis", -1), epsilon=a.get("epsilon", 1e-5)),
    "Gather": lambda a, i: np.take(i[0], i[1].astype(np.int64), axis=a.get("axis", 0)),
    "Reshape": lambda a, i: i[0].reshape([int(d) if d != 0 else i[0].shape[k] for k, d in enumerate(i[1])]),
    "Transpose": lambda a, i: np.transpose(i[0], a.get("perm")), "Concat": lambda a, i: np.concatenate(i, axis=a.get("axis", 0)),
    "Constant": lambda a, i: a["value"], "Sqrt": lambda a, i: np.sqrt(i[0]), "Pow": lambda a, i: i[0] ** i[1],
    "ReduceMean": lambda a, i: i[0].mean(axis=tuple(a.get("axes", [-1])), keepdims=bool(a.get("keepdims", 1))),
    "QuantizeLinear": lambda a, i: np.clip(np.round(i[0] / i[1]) + (i[2] if len(i) > 2 else 0), -128, 127).astype(np.int8),
    "DequantizeLinear": lambda a, i: (i[0].astype(np.float32) - (i[2] if len(i) > 2 else 0)) * i[1],
}


def _eval_node(n: "Node", env: dict) -> None:
    """Runs one node on ``env``. Empty input names are optional inputs that were left out (passed as None unless they
    trail); an operator returns one array, or a tuple that is bound to the node's outputs in order."""
    ins = [env[i] if i else None for i in n.inputs]
    while ins and ins[-1] is None:
        ins.pop()
    attrs = n.attrs if len(n.outputs) <= 1 else dict(n.attrs, _n_outputs=len(n.outputs))
    out = OPS[n.op_type](attrs, ins)
    if isinstance(out, tuple):
        for name, val in zip(n.outputs, out):
            if name:
                env[name] = val
    else:
        env[n.outputs[0]] = out


def run_model(m: Model, feeds: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    env = dict(m.graph.initializers)
    env.update(feeds)
    for n in m.graph.nodes:
        _eval_node(n, env)
    return {o.name: env[o.name] for o in m.graph.outputs}


def infer_shapes(m: Model, input_shapes: Optional[Dict[str, tuple]] = None) -> Dict[str, tuple]:
    """Shapes by abstract execution on zero tensors (exact for the supported op set)."""
    feeds = {}
    for i in m.graph.inputs:
        shp = (input_shapes or {}).get(i.name, tuple(d if isinstance(d, int) and d > 0 else 1 for d in i.shape))
        feeds[i.name] = np.zeros(shp, dtype=_NP.get(i.dtype, np.float32))
    env = dict(m.graph.initializers)
    env.update(feeds)
    shapes = {k: tuple(v.shape) for k, v in env.items()}
    for n in m.graph.nodes:
        _eval_node(n, env)
        for o in n.outputs:
            if o in env:
                shapes[o] = tuple(np.shape(env[o]))
    return shapes


def optimize(m: Model) -> Model:
    """Fold nodes whose inputs are all constants; drop nodes whose outputs nobody uses."""
    g = m.graph
    const = dict(g.initializers)
    kept = []
    for n in g.nodes:
        if n.op_type in OPS and all((i in const) for i in n.inputs if i) and (n.inputs or n.op_type == "Constant"):
            _eval_node(n, const)
            for o in n.outputs:
                if o in const:
                    const[o] = np.asarray(const[o])
        else:
            kept.append(n)
    needed = {o.name for o in g.outputs}
    live = []
    for n in reversed(kept):
        if any(o in needed for o in n.outputs):
            live.append(n)
            needed.update(i for i in n.inputs if i)
    live.reverse()
    inits = {k: v for k, v in const.items() if k in needed}
    return Model(Graph(live, g.inputs, g.outputs, inits, g.name), m.ir_version, m.opset, m.producer)


def quantize_qdq(m: Model) -> Model:
    """Weight-only QDQ: every 2-D float initialiser feeding MatMul / Gemm becomes int8 + DequantizeLinear."""
    g = m.graph
    inits, nodes = dict(g.initializers), []
    for n in g.nodes:
        if n.op_type in ("MatMul", "Gemm") and len(n.inputs) > 1 and n.inputs[1] in inits and inits[n.inputs[1]].ndim == 2:
            w = inits.pop(n.inputs[1])
            s = np.float32(max(np.abs(w).max() / 127.0, 1e-12))
            q = np.clip(np.round(w / s), -127, 127).astype(np.int8)
            inits[n.inputs[1] + "_q"], inits[n.inputs[1] + "_scale"] = q, np.array(s, dtype=np.float32)
            nodes.append(Node("DequantizeLinear", [n.inputs[1] + "_q", n.inputs[1] + "_scale"], [n.inputs[1] + "_dq"]))
            n = Node(n.op_type, [n.inputs[0], n.inputs[1] + "_dq"] + n.inputs[2:], n.outputs, n.attrs, n.name)
        nodes.append(n)
    return Model(Graph(nodes, g.inputs, g.outputs, inits, g.name), m.ir_version, m.opset, m.producer)


# ----------------------------------------------------------------------------- export from torch
def export_module(module, example_input, path: Optional[str] = None) -> Model:
    """Feed-forward stacks of Linear / LayerNorm / activations / Embedding (Sequential-like modules)."""
    import torch
    import torch.nn as tnn
    g = Graph(inputs=[ValueInfo("input", DT_INT64 if example_input.dtype == torch.int64 else DT_FLOAT,
                                ("batch",) + tuple(example_input.shape[1:]))])
    cur, k = "input", 0

    def emit(op, ins, attrs=None):
        nonlocal cur, k
        out = f"v{k}"
        k += 1
        g.nodes.append(Node(op, ins, [out], attrs or {}, f"{op}_{k}"))
        cur = out

    leaves = [mod for mod in module.modules() if not list(mod.children())]
    for mod in leaves:
        name = f"p{k}"
        if hasattr(mod, "weight") and mod.weight is not None and mod.weight.dim() == 2 and hasattr(mod, "in_features"):
            g.initializers[name + "_w"] = mod.weight.detach().float().t().contiguous().numpy()
            emit("MatMul", [cur, name + "_w"])
            if getattr(mod, "bias", None) is not None:
                g.initializers[name + "_b"] = mod.bias.detach().float().numpy()
                emit("Add", [cur, name + "_b"])
        elif isinstance(mod, tnn.Embedding) or type(mod).__name__ == "Embedding":
            g.initializers[name + "_w"] = mod.weight.detach().float().numpy()
            emit("Gather", [name + "_w", cur], {"axis": 0})
        elif type(mod).__name__ == "LayerNorm":
            g.initializers[name + "_w"] = mod.weight.detach().float().numpy()
            g.initializers[name + "_b"] = mod.bias.detach().float().numpy()
            emit("LayerNormalization", [cur, name + "_w", name + "_b"], {"axis": -1, "epsilon": float(mod.eps)})
        elif type(mod).__name__ in ("ReLU", "Sigmoid", "Tanh", "GELU"):
            emit({"ReLU": "Relu", "GELU": "Gelu"}.get(type(mod).__name__, type(mod).__name__), [cur])
        elif type(mod).__name__ in ("Dropout", "Identity"):
            continue
        else:
            raise NotImplementedError(f"export of {type(mod).__name__}")
    g.outputs = [ValueInfo(cur, DT_FLOAT, ())]
    m = Model(g)
    if path:
        m.save(path)
    return m


# ----------------------------------------------------------------------------- external data / runtime adapter
def save_external_data(m: Model, path: str, data_file: Optional[str] = None, size_threshold: int = 1024) -> List[str]:
    """Writes ``path`` with every initializer of at least ``size_threshold`` bytes moved into one side file
    (``<model name>.data`` beside it unless named), 64-byte aligned, referenced by location / offset / length as in
    the ONNX external-data convention (the reference's onnx/external_data.py:26-55). Returns the moved names."""
    import os
    data_file = data_file or os.path.basename(path) + ".data"
    if os.path.basename(data_file) != data_file:
        raise ValueError("the data file must sit beside the model (a plain file name)")
    moved, ext, off = [], {}, 0
    with open(os.path.join(os.path.dirname(os.path.abspath(path)), data_file), "wb") as f:
        for name, arr in m.graph.initializers.items():
            raw = np.ascontiguousarray(arr).tobytes()
            if len(raw) < size_threshold:
                continue
            pad = (-off) % 64
            f.write(b"\x00" * pad)
            off += pad
            f.write(raw)
            ext[name] = {"location": data_file, "offset": str(off), "length": str(len(raw))}
            off += len(raw)
            moved.append(name)
    out = Model(m.graph, m.ir_version, m.opset, m.producer, ext)
    out.save(path)
    return moved


def load_external_data(path: str, base_dir: Optional[str] = None) -> Model:
    """Loads a model and pulls every external initializer in from its side file. File names are taken relative to the
    model's folder (or ``base_dir``) and may not leave it; offsets and lengths are checked against the file and the
    tensor's shape (onnx/external_data.py:92-95 of the reference trusts them)."""
    import os
    m = Model.load(path)
    base = os.path.abspath(base_dir or os.path.dirname(os.path.abspath(path)))
    for name, e in m.external.items():
        loc = e.get("location", "")
        full = os.path.abspath(os.path.join(base, loc))
        if not loc or os.path.isabs(loc) or os.path.commonpath([base, full]) != base:
            raise ValueError(f"external data of {name!r} points outside the model folder: {loc!r}")
        arr = m.graph.initializers[name]
        off, want = int(e.get("offset", 0)), arr.size * arr.dtype.itemsize
        length = int(e.get("length", want))
        if off < 0 or length != want or off + length > os.path.getsize(full):
            raise ValueError(f"external data of {name!r}: offset {off} / length {length} do not fit the file or the shape")
        with open(full, "rb") as f:
            f.seek(off)
            m.graph.initializers[name] = np.frombuffer(f.read(length), dtype=arr.dtype).reshape(arr.shape).copy()
    m.external = {}
    return m


def has_onnxruntime() -> bool:
    try:
        import onnxruntime  # noqa: F401
        return True
    except Exception:  # noqa: BLE001
        return False


class OnnxRuntimeSession:
    """``InferenceSession``-shaped front: runs on onnxruntime when it is installed (or when ``require_ort``), else on
    this toolkit's own executor, with the same ``get_inputs`` / ``get_outputs`` / ``run`` surface
    (onnx/runtime/ort_adapter.py:38-73 of the reference)."""

    def __init__(self, model: Model, require_ort: bool = False):
        self.model, self._sess = model, None
        if has_onnxruntime():
            import onnxruntime as ort
            self._sess = ort.InferenceSession(model.serialize(), providers=["CPUExecutionProvider"])
        elif require_ort:
            raise RuntimeError("onnxruntime is not installed")
        self.backend = "onnxruntime" if self._sess is not None else "sneppx"

    def get_inputs(self) -> List[ValueInfo]:
        return list(self.model.graph.inputs)

    def get_outputs(self) -> List[ValueInfo]:
        return list(self.model.graph.outputs)

    def run(self, output_names: Optional[List[str]], inputs: Dict[str, np.ndarray]) -> List[np.ndarray]:
        if self._sess is not None:
            return self._sess.run(output_names, inputs)
        res = run_model(self.model, inputs)
        names = output_names or [o.name for o in self.model.graph.outputs]
        return [res[n] for n in names]


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(prog="sneppx-onnx")
    ap.add_argument("command", choices=["check", "shapes", "optimize", "quantize", "info"])
    ap.add_argument("model")
    ap.add_argument("-o", "--output")
    a = ap.parse_args(argv)
    m = Model.load(a.model)
    if a.command == "check":
        errs = check_model(m)
        print("OK" if not errs else "\n".join(errs))
        return 1 if errs else 0
    if a.command == "shapes":
        for k, v in infer_shapes(m).items():
            print(k, v)
    elif a.command == "info":
        print(f"ir {m.ir_version} opset {m.opset} nodes {len(m.graph.nodes)} initializers {len(m.graph.initializers)}")
    else:
        out = optimize(m) if a.command == "optimize" else quantize_qdq(m)
        out.save(a.output or a.model.replace(".onnx", f".{a.command}.onnx"))
    return 0
