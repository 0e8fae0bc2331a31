"""More of the ONNX operator set for the NumPy executor of ``toolkit.py``, graph passes, a stricter checker and an
exporter for convolutional stacks.

Importing this module registers the operators in ``toolkit.OPS``. An operator function takes ``(attrs, inputs)`` and
returns one array, or a tuple of arrays for multi-output nodes (``Split``, ``TopK``); ``toolkit.run_model`` binds
them to the node's output names in order. Reference modules of the same purpose: onnx/onnx_export.py (operator
emitters and the export walker), onnx/onnx_check.py (per-operator attribute checks), onnx/graph_optimizer.py.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import toolkit as tk
from .toolkit import DT_FLOAT, DT_INT64, Graph, Model, Node, ValueInfo

_ONNX_TO_NP = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16,
               11: np.float64, 12: np.uint32, 13: np.uint64}


def _axes(a, i, pos=1, default=None):
    """Axes from the attribute (opset < 13/18) or from the optional input at ``pos`` (later opsets)."""
    if "axes" in a:
        return tuple(int(x) for x in a["axes"])
    if len(i) > pos and i[pos] is not None and np.size(i[pos]):
        return tuple(int(x) for x in np.asarray(i[pos]).reshape(-1))
    return default


def _reduce(fn):
    def op(a, i):
        ax = _axes(a, i)
        if ax is None and a.get("noop_with_empty_axes", 0):
            return i[0]
        return fn(i[0], axis=ax, keepdims=bool(a.get("keepdims", 1)))
    return op


def _pads(a, nd):
    p = list(a.get("pads", [0] * (2 * nd)))
    return [(int(p[k]), int(p[k + nd])) for k in range(nd)]


def _auto_pad(a, in_shape, kernel, strides, dilations):
    mode = a.get("auto_pad", "NOTSET")
    nd = len(kernel)
    if mode in ("NOTSET", "", None):
        return _pads(a, nd)
    if mode == "VALID":
        return [(0, 0)] * nd
    out = []
    for k in range(nd):
        o = math.ceil(in_shape[k] / strides[k])
        total = max((o - 1) * strides[k] + (kernel[k] - 1) * dilations[k] + 1 - in_shape[k], 0)
        lo = total // 2 if mode == "SAME_UPPER" else total - total // 2
        out.append((lo, total - lo))
    return out


def _windows(x, kernel, strides, dilations, pads, fill=0.0, ceil_mode=0):
    """Sliding windows of an [N, C, *spatial] array as [N, C, *out, *kernel] (a strided view of the padded copy)."""
    nd = len(kernel)
    if ceil_mode:
        pads = list(pads)
        for k in range(nd):
            span = x.shape[2 + k] + pads[k][0] + pads[k][1] - ((kernel[k] - 1) * dilations[k] + 1)
            if span % strides[k]:
                pads[k] = (pads[k][0], pads[k][1] + strides[k] - span % strides[k])
    xp = np.pad(x, [(0, 0), (0, 0)] + list(pads), constant_values=fill)
    out = [(xp.shape[2 + k] - ((kernel[k] - 1) * dilations[k] + 1)) // strides[k] + 1 for k in range(nd)]
    s = xp.strides
    shape = list(xp.shape[:2]) + out + list(kernel)
    strides_ = list(s[:2]) + [s[2 + k] * strides[k] for k in range(nd)] + [s[2 + k] * dilations[k] for k in range(nd)]
    return np.lib.stride_tricks.as_strided(xp, shape, strides_, writeable=False)


def _conv(a, i):
    x, w = i[0], i[1]
    b = i[2] if len(i) > 2 else None
    nd = x.ndim - 2
    kernel = list(a.get("kernel_shape", w.shape[2:]))
    strides = list(a.get("strides", [1] * nd))
    dil = list(a.get("dilations", [1] * nd))
    groups = int(a.get("group", 1))
    win = _windows(x, kernel, strides, dil, _auto_pad(a, x.shape[2:], kernel, strides, dil))   # [N, C, *out, *k]
    N, C = x.shape[:2]
    M = w.shape[0]
    out_sp = win.shape[2: 2 + nd]
    win = win.reshape(N, groups, C // groups, *out_sp, *kernel)
    wg = w.reshape(groups, M // groups, C // groups, *kernel)
    sp = "xyz"[:nd]
    ks = "uvw"[:nd]
    y = np.einsum(f"ngc{sp}{ks},gmc{ks}->ngm{sp}", win, wg, optimize=True).reshape(N, M, *out_sp)
    if b is not None:
        y = y + b.reshape(1, -1, *([1] * nd))
    return y.astype(x.dtype)


def _pool(kind):
    def op(a, i):
        x = i[0]
        nd = x.ndim - 2
        kernel = list(a["kernel_shape"])
        strides = list(a.get("strides", [1] * nd))
        dil = list(a.get("dilations", [1] * nd))
        pads = _auto_pad(a, x.shape[2:], kernel, strides, dil)
        axes = tuple(range(2 + nd, 2 + 2 * nd))
        if kind == "max":
            return _windows(x, kernel, strides, dil, pads, -np.inf, a.get("ceil_mode", 0)).max(axis=axes).astype(x.dtype)
        win = _windows(x, kernel, strides, dil, pads, 0.0, a.get("ceil_mode", 0))
        if a.get("count_include_pad", 0):
            return win.mean(axis=axes).astype(x.dtype)
        ones = _windows(np.ones_like(x), kernel, strides, dil, pads, 0.0, a.get("ceil_mode", 0))
        return (win.sum(axis=axes) / np.maximum(ones.sum(axis=axes), 1)).astype(x.dtype)
    return op


def _batchnorm(a, i):
    x, scale, bias, mean, var = i[:5]
    shp = [1, -1] + [1] * (x.ndim - 2)
    return ((x - mean.reshape(shp)) / np.sqrt(var.reshape(shp) + a.get("epsilon", 1e-5)) * scale.reshape(shp) +
            bias.reshape(shp)).astype(x.dtype)


def _slice(a, i):
    x = i[0]
    if "starts" in a:      # opset < 10: attributes
        starts, ends, axes, steps = a["starts"], a["ends"], a.get("axes"), None
    else:
        starts, ends = i[1], i[2]
        axes = i[3] if len(i) > 3 else None
        steps = i[4] if len(i) > 4 else None
    axes = list(range(len(starts))) if axes is None else [int(v) for v in np.asarray(axes).reshape(-1)]
    steps = [1] * len(axes) if steps is None else [int(v) for v in np.asarray(steps).reshape(-1)]
    sl = [slice(None)] * x.ndim
    for st, en, ax, sp in zip(np.asarray(starts).reshape(-1), np.asarray(ends).reshape(-1), axes, steps):
        st, en = int(np.clip(st, -(2 ** 62), 2 ** 62)), int(np.clip(en, -(2 ** 62), 2 ** 62))
        sl[ax] = slice(st, en, sp)
    return x[tuple(sl)]


def _split(a, i):
    x = i[0]
    axis = int(a.get("axis", 0))
    if len(i) > 1 and i[1] is not None:
        sizes = [int(v) for v in np.asarray(i[1]).reshape(-1)]
    elif "split" in a:
        sizes = [int(v) for v in a["split"]]
    else:
        n = int(a.get("num_outputs", a.get("_n_outputs", 2)))
        base = -(-x.shape[axis] // n)
        sizes = [min(base, x.shape[axis] - k * base) for k in range(n)]
    return tuple(np.split(x, np.cumsum(sizes)[:-1], axis=axis))


def _topk(a, i):
    x, k = i[0], int(np.asarray(i[1]).reshape(-1)[0])
    axis, largest = int(a.get("axis", -1)), int(a.get("largest", 1))
    order = np.argsort(-x if largest else x, axis=axis, kind="stable")
    idx = np.take(order, np.arange(k), axis=axis)
    return np.take_along_axis(x, idx, axis=axis), idx.astype(np.int64)


def _squeeze(a, i):
    ax = _axes(a, i)
    return np.squeeze(i[0], axis=ax) if ax is not None else np.squeeze(i[0])


def _unsqueeze(a, i):
    x = i[0]
    for ax in sorted(int(v) % (x.ndim + len(_axes(a, i))) for v in _axes(a, i)):
        x = np.expand_dims(x, ax)
    return x


def _pad(a, i):
    x = i[0]
    pads = a["pads"] if "pads" in a else [int(v) for v in np.asarray(i[1]).reshape(-1)]
    value = a.get("value", 0.0) if len(i) < 3 or i[2] is None else float(np.asarray(i[2]).reshape(-1)[0])
    nd = x.ndim
    width = [(int(pads[k]), int(pads[k + nd])) for k in range(nd)]
    mode = {"constant": "constant", "reflect": "reflect", "edge": "edge"}[a.get("mode", "constant")]
    return np.pad(x, width, mode=mode, **({"constant_values": value} if mode == "constant" else {}))


def _erf(x):
    # Abramowitz-Stegun 7.1.26 is too coarse for GELU parity; use the series / continued fraction split of math.erf
    return np.vectorize(math.erf, otypes=[x.dtype if x.dtype.kind == "f" else np.float32])(x)


def _rmsnorm(a, i):
    x, w = i[0], i[1]
    ax = int(a.get("axis", -1))
    return (x / np.sqrt((x.astype(np.float32) ** 2).mean(axis=ax, keepdims=True) + a.get("epsilon", 1e-5)) * w).astype(x.dtype)


def _logsoftmax(a, i):
    ax = a.get("axis", -1)
    z = i[0] - i[0].max(axis=ax, keepdims=True)
    return z - np.log(np.exp(z).sum(axis=ax, keepdims=True))


def _expand(a, i):
    shape = [int(v) for v in np.asarray(i[1]).reshape(-1)]
    return i[0] * np.ones(shape, dtype=i[0].dtype)


def _range(a, i):
    s, l, d = (np.asarray(v).reshape(-1)[0] for v in i[:3])
    return np.arange(s, l, d).astype(np.asarray(i[0]).dtype)


def _flatten(a, i):
    ax = int(a.get("axis", 1))
    x = i[0]
    return x.reshape(int(np.prod(x.shape[:ax], dtype=np.int64)) if ax else 1, -1)


def _clip(a, i):
    lo = a.get("min") if len(i) < 2 or i[1] is None else i[1]
    hi = a.get("max") if len(i) < 3 or i[2] is None else i[2]
    return np.clip(i[0], lo, hi)


EXTRA_OPS = {
    "Conv": _conv, "MaxPool": _pool("max"), "AveragePool": _pool("avg"),
    "GlobalAveragePool": lambda a, i: i[0].mean(axis=tuple(range(2, i[0].ndim)), keepdims=True),
    "GlobalMaxPool": lambda a, i: i[0].max(axis=tuple(range(2, i[0].ndim)), keepdims=True),
    "BatchNormalization": _batchnorm, "Slice": _slice, "Split": _split, "TopK": _topk, "Squeeze": _squeeze,
    "Unsqueeze": _unsqueeze, "Pad": _pad, "Flatten": _flatten, "Clip": _clip, "Expand": _expand, "Range": _range,
    "Cast": lambda a, i: i[0].astype(_ONNX_TO_NP[int(a["to"])]),
    "Shape": lambda a, i: np.array(i[0].shape, dtype=np.int64),
    "Size": lambda a, i: np.array(i[0].size, dtype=np.int64),
    "Where": lambda a, i: np.where(i[0], i[1], i[2]),
    "Equal": lambda a, i: i[0] == i[1], "Less": lambda a, i: i[0] < i[1], "Greater": lambda a, i: i[0] > i[1],
    "LessOrEqual": lambda a, i: i[0] <= i[1], "GreaterOrEqual": lambda a, i: i[0] >= i[1],
    "Not": lambda a, i: ~i[0].astype(bool), "And": lambda a, i: i[0] & i[1], "Or": lambda a, i: i[0] | i[1],
    "Exp": lambda a, i: np.exp(i[0]), "Log": lambda a, i: np.log(i[0]), "Neg": lambda a, i: -i[0], "Abs": lambda a, i: np.abs(i[0]),
    "Reciprocal": lambda a, i: 1.0 / i[0], "Floor": lambda a, i: np.floor(i[0]), "Ceil": lambda a, i: np.ceil(i[0]),
    "Erf": lambda a, i: _erf(i[0]), "Min": lambda a, i: np.minimum.reduce(i), "Max": lambda a, i: np.maximum.reduce(i),
    "Sum": lambda a, i: np.add.reduce(i), "Mean": lambda a, i: np.add.reduce(i) / len(i),
    "LeakyRelu": lambda a, i: np.where(i[0] >= 0, i[0], a.get("alpha", 0.01) * i[0]),
    "Elu": lambda a, i: np.where(i[0] >= 0, i[0], a.get("alpha", 1.0) * (np.exp(np.minimum(i[0], 0)) - 1)),
    "Softplus": lambda a, i: np.logaddexp(i[0], 0), "HardSigmoid": lambda a, i: np.clip(a.get("alpha", 0.2) * i[0] + a.get("beta", 0.5), 0, 1),
    "Swish": lambda a, i: i[0] / (1 + np.exp(-i[0])), "LogSoftmax": _logsoftmax,
    "SimplifiedLayerNormalization": _rmsnorm, "RMSNormalization": _rmsnorm,
    "ReduceSum": _reduce(np.sum), "ReduceMax": _reduce(np.max), "ReduceMin": _reduce(np.min), "ReduceProd": _reduce(np.prod),
    "ReduceL2": lambda a, i: np.sqrt(_reduce(np.sum)(a, [i[0] ** 2] + list(i[1:]))),
    "ArgMax": lambda a, i: (np.expand_dims(np.argmax(i[0], axis=a.get("axis", 0)), a.get("axis", 0)) if a.get("keepdims", 1)
                            else np.argmax(i[0], axis=a.get("axis", 0))).astype(np.int64),
    "ArgMin": lambda a, i: (np.expand_dims(np.argmin(i[0], axis=a.get("axis", 0)), a.get("axis", 0)) if a.get("keepdims", 1)
                            else np.argmin(i[0], axis=a.get("axis", 0))).astype(np.int64),
    "Tile": lambda a, i: np.tile(i[0], [int(v) for v in np.asarray(i[1]).reshape(-1)]),
    "Einsum": lambda a, i: np.einsum(a["equation"], *i),
    "CumSum": lambda a, i: np.cumsum(i[0], axis=int(np.asarray(i[1]).reshape(-1)[0])),
    "Trilu": lambda a, i: (np.triu if a.get("upper", 1) else np.tril)(i[0], int(np.asarray(i[1]).reshape(-1)[0]) if len(i) > 1 else 0),
    "GatherElements": lambda a, i: np.take_along_axis(i[0], i[1].astype(np.int64), axis=a.get("axis", 0)),
    "ConstantOfShape": lambda a, i: np.full([int(v) for v in np.asarray(i[0]).reshape(-1)],
                                            np.asarray(a.get("value", np.zeros(1, np.float32))).reshape(-1)[0]),
    "Dropout": lambda a, i: i[0],
}
# ReduceMean of the base table ignores the axes-as-input form of later opsets
EXTRA_OPS["ReduceMean"] = _reduce(np.mean)
tk.OPS.update(EXTRA_OPS)


# ----------------------------------------------------------------------------- graph passes
def _consumers(g: Graph) -> Dict[str, List[Node]]:
    use: Dict[str, List[Node]] = {}
    for n in g.nodes:
        for i in n.inputs:
            if i:
                use.setdefault(i, []).append(n)
    return use


def _rename_input(g: Graph, old: str, new: str) -> None:
    for n in g.nodes:
        n.inputs = [new if i == old else i for i in n.inputs]
    for o in g.outputs:
        if o.name == old:
            o.name = new


def eliminate_identity(m: Model) -> int:
    """Removes Identity / Dropout nodes (inference graph) by rewiring their consumers. Returns the number removed."""
    g, removed = m.graph, 0
    outs = {o.name for o in g.outputs}
    for n in list(g.nodes):
        if n.op_type in ("Identity", "Dropout") and n.outputs[0] not in outs:
            _rename_input(g, n.outputs[0], n.inputs[0])
            g.nodes.remove(n)
            removed += 1
    return removed


def fuse_matmul_add(m: Model) -> int:
    """MatMul by a 2-D constant followed by Add of a 1-D constant -> one Gemm (only when the activation is 2-D, which
    shape inference must confirm; otherwise the pair is left alone)."""
    g = m.graph
    shapes = tk.infer_shapes(m)
    use, fused = _consumers(g), 0
    for n in list(g.nodes):
        if n.op_type != "MatMul" or n.inputs[1] not in g.initializers or g.initializers[n.inputs[1]].ndim != 2:
            continue
        if len(shapes.get(n.inputs[0], ())) != 2:
            continue
        cs = use.get(n.outputs[0], [])
        if len(cs) != 1 or cs[0].op_type != "Add":
            continue
        add = cs[0]
        other = add.inputs[1] if add.inputs[0] == n.outputs[0] else add.inputs[0]
        if other not in g.initializers or g.initializers[other].ndim != 1:
            continue
        idx = g.nodes.index(n)
        g.nodes[idx] = Node("Gemm", [n.inputs[0], n.inputs[1], other], list(add.outputs), {"alpha": 1.0, "beta": 1.0}, n.name or "gemm")
        g.nodes.remove(add)
        fused += 1
    return fused


def fuse_transposes(m: Model) -> int:
    """Two Transposes in a row become one (or none when the permutations cancel)."""
    g, changed = m.graph, 0
    outs = {o.name for o in g.outputs}
    produced = {o: n for n in g.nodes for o in n.outputs}
    for n in list(g.nodes):
        if n.op_type != "Transpose" or n not in g.nodes:
            continue
        p = produced.get(n.inputs[0])
        if p is None or p.op_type != "Transpose" or p.outputs[0] in outs or len(_consumers(g).get(p.outputs[0], [])) != 1:
            continue
        p1, p2 = list(p.attrs["perm"]), list(n.attrs["perm"])
        perm = [p1[k] for k in p2]
        g.nodes.remove(p)
        if perm == list(range(len(perm))) and n.outputs[0] not in outs:
            _rename_input(g, n.outputs[0], p.inputs[0])
            g.nodes.remove(n)
        else:
            n.inputs, n.attrs = [p.inputs[0]], {"perm": perm}
        changed += 1
    return changed


def fold_batchnorm_into_conv(m: Model) -> int:
    """Conv with constant weights followed only by BatchNormalization with constant statistics -> one Conv."""
    g, folded = m.graph, 0
    use = _consumers(g)
    for n in list(g.nodes):
        if n.op_type != "Conv" or n.inputs[1] not in g.initializers:
            continue
        cs = use.get(n.outputs[0], [])
        if len(cs) != 1 or cs[0].op_type != "BatchNormalization" or any(i not in g.initializers for i in cs[0].inputs[1:5]):
            continue
        bn = cs[0]
        scale, bias, mean, var = (g.initializers[i].astype(np.float64) for i in bn.inputs[1:5])
        k = scale / np.sqrt(var + bn.attrs.get("epsilon", 1e-5))
        w = g.initializers[n.inputs[1]]
        b = g.initializers[n.inputs[2]].astype(np.float64) if len(n.inputs) > 2 and n.inputs[2] else np.zeros(w.shape[0])
        wn, bn_ = n.inputs[1] + "_bn", (n.inputs[2] if len(n.inputs) > 2 and n.inputs[2] else n.inputs[1]) + "_bnb"
        g.initializers[wn] = (w * k.reshape(-1, *([1] * (w.ndim - 1)))).astype(w.dtype)
        g.initializers[bn_] = ((b - mean) * k + bias).astype(w.dtype)
        n.inputs = [n.inputs[0], wn, bn_]
        n.outputs = list(bn.outputs)
        g.nodes.remove(bn)
        folded += 1
    return folded


def eliminate_common_subexpressions(m: Model) -> int:
    """Nodes with the same operator, inputs and attributes compute the same value: keep the first."""
    g, seen, removed = m.graph, {}, 0
    outs = {o.name for o in g.outputs}
    for n in list(g.nodes):
        key = (n.op_type, tuple(n.inputs), repr(sorted((k, np.asarray(v).tolist()) for k, v in n.attrs.items())))
        first = seen.get(key)
        if first is None or len(n.outputs) != 1 or n.outputs[0] in outs:
            seen.setdefault(key, n)
            continue
        _rename_input(g, n.outputs[0], first.outputs[0])
        g.nodes.remove(n)
        removed += 1
    return removed


def run_passes(m: Model, passes: Optional[Sequence[str]] = None) -> Dict[str, int]:
    """Applies the named passes until none of them changes the graph; then constant folding / dead-code removal of
    ``toolkit.optimize``. Returns how often each pass fired; the optimised model replaces ``m.graph`` in place."""
    table = {"identity": eliminate_identity, "transposes": fuse_transposes, "bn_fold": fold_batchnorm_into_conv,
             "gemm": fuse_matmul_add, "cse": eliminate_common_subexpressions}
    names = list(passes) if passes is not None else list(table)
    counts = {k: 0 for k in names}
    for _ in range(16):
        fired = 0
        for k in names:
            c = table[k](m)
            counts[k] += c
            fired += c
        if not fired:
            break
    m.graph = tk.optimize(m).graph
    return counts


def topological_sort(m: Model) -> None:
    """Reorders the nodes so that every value is produced before it is used (raises ValueError on a cycle)."""
    g = m.graph
    known = set(g.initializers) | {i.name for i in g.inputs}
    todo, order = list(g.nodes), []
    while todo:
        ready = [n for n in todo if all((not i) or i in known for i in n.inputs)]
        if not ready:
            raise ValueError("graph has a cycle or uses undefined values: " + ", ".join(sorted({i for n in todo for i in n.inputs if i and i not in known})[:5]))
        for n in ready:
            order.append(n)
            known.update(o for o in n.outputs if o)
            todo.remove(n)
    g.nodes = order


# ----------------------------------------------------------------------------- stricter checker
_ARITY = {"MatMul": (2, 2), "Gemm": (2, 3), "Conv": (2, 3), "BatchNormalization": (5, 5), "Add": (2, 2), "Sub": (2, 2), "Mul": (2, 2),
          "Div": (2, 2), "Where": (3, 3), "Gather": (2, 2), "Reshape": (2, 2), "LayerNormalization": (2, 3), "Relu": (1, 1),
          "Transpose": (1, 1), "Softmax": (1, 1), "Cast": (1, 1), "TopK": (2, 2), "Split": (1, 2), "Slice": (1, 5), "Pad": (1, 4)}
_REQUIRED_ATTRS = {"Cast": ("to",), "MaxPool": ("kernel_shape",), "AveragePool": ("kernel_shape",), "Einsum": ("equation",)}


def check_model_strict(m: Model) -> List[str]:
    """``toolkit.check_model`` plus: operator arity, required attributes, attribute value checks (permutations, pads
    and strides of the right length, Cast targets), duplicate node names, opset sanity, shape inference as a last
    consistency check (an executor error on zero tensors is reported with the node that raised it)."""
    errs = tk.check_model(m)
    if not 7 <= m.opset <= 23:
        errs.append(f"opset {m.opset} outside the supported range 7..23")
    names = [n.name for n in m.graph.nodes if n.name]
    for d in sorted({x for x in names if names.count(x) > 1}):
        errs.append(f"node name '{d}' used more than once")
    for n in m.graph.nodes:
        tag = n.name or n.op_type
        lo_hi = _ARITY.get(n.op_type)
        if lo_hi and not lo_hi[0] <= len(n.inputs) <= lo_hi[1]:
            errs.append(f"{tag}: {len(n.inputs)} inputs, expected {lo_hi[0]}..{lo_hi[1]}")
        for a in _REQUIRED_ATTRS.get(n.op_type, ()):
            if a not in n.attrs:
                errs.append(f"{tag}: required attribute '{a}' is missing")
        if n.op_type == "Transpose" and "perm" in n.attrs and sorted(n.attrs["perm"]) != list(range(len(n.attrs["perm"]))):
            errs.append(f"{tag}: perm {list(n.attrs['perm'])} is not a permutation")
        if n.op_type == "Cast" and "to" in n.attrs and int(n.attrs["to"]) not in _ONNX_TO_NP:
            errs.append(f"{tag}: unknown Cast target {n.attrs['to']}")
        if n.op_type in ("Conv", "MaxPool", "AveragePool") and "kernel_shape" in n.attrs:
            nd = len(n.attrs["kernel_shape"])
            for a, want in (("strides", nd), ("dilations", nd), ("pads", 2 * nd)):
                if a in n.attrs and len(n.attrs[a]) != want:
                    errs.append(f"{tag}: {a} has {len(n.attrs[a])} entries, expected {want}")
            if any(int(k) <= 0 for k in n.attrs["kernel_shape"]):
                errs.append(f"{tag}: non-positive kernel size")
    if not errs:
        try:
            tk.infer_shapes(m)
        except Exception as e:  # noqa: BLE001  (whatever the executor raises on this graph is the finding)
            errs.append(f"shape inference failed: {type(e).__name__}: {e}")
    return errs


# ----------------------------------------------------------------------------- exporter for convolutional stacks
def export_sequential(module, example_input, path: Optional[str] = None) -> Model:
    """Exports a feed-forward stack (``torch.nn.Sequential``-like: leaves are applied in registration order) of Conv2d /
    BatchNorm2d (eval statistics) / pooling / Flatten / Linear / LayerNorm / RMSNorm / Embedding / activations."""
    import torch
    g = Graph(inputs=[ValueInfo("input", DT_INT64 if example_input.dtype == torch.int64 else DT_FLOAT,
                                ("batch",) + tuple(example_input.shape[1:]))])
    cur, k = "input", 0

    def emit(op, ins, attrs=None):
        nonlocal cur, k
        out = f"v{k}"
        k += 1
        g.nodes.append(Node(op, ins, [out], attrs or {}, f"{op}_{k}"))
        cur = out

    def const(name, t):
        g.initializers[name] = t.detach().float().cpu().numpy() if hasattr(t, "detach") else np.asarray(t)
        return name

    def pair(v):
        return [int(v), int(v)] if isinstance(v, int) else [int(x) for x in v]

    for mod in [x for x in module.modules() if not list(x.children())]:
        t, p = type(mod).__name__, f"p{k}"
        if t == "Conv2d":
            pads = pair(mod.padding) if not isinstance(mod.padding, str) else None
            attrs = {"kernel_shape": pair(mod.kernel_size), "strides": pair(mod.stride), "dilations": pair(mod.dilation),
                     "group": int(mod.groups)}
            if pads is not None:
                attrs["pads"] = pads + pads
            else:
                attrs["auto_pad"] = {"same": "SAME_UPPER", "valid": "VALID"}[mod.padding]
            ins = [cur, const(p + "_w", mod.weight)] + ([const(p + "_b", mod.bias)] if mod.bias is not None else [])
            emit("Conv", ins, attrs)
        elif t == "BatchNorm2d":
            emit("BatchNormalization", [cur, const(p + "_s", mod.weight), const(p + "_b", mod.bias),
                                        const(p + "_m", mod.running_mean), const(p + "_v", mod.running_var)], {"epsilon": float(mod.eps)})
        elif t in ("MaxPool2d", "AvgPool2d"):
            ks = pair(mod.kernel_size)
            pads = pair(mod.padding)
            attrs = {"kernel_shape": ks, "strides": pair(mod.stride if mod.stride is not None else mod.kernel_size),
                     "pads": pads + pads, "ceil_mode": int(mod.ceil_mode)}
            if t == "AvgPool2d":
                attrs["count_include_pad"] = int(mod.count_include_pad)
            emit("MaxPool" if t == "MaxPool2d" else "AveragePool", [cur], attrs)
        elif t == "AdaptiveAvgPool2d" and pair(mod.output_size) == [1, 1]:
            emit("GlobalAveragePool", [cur])
        elif t == "Flatten":
            emit("Flatten", [cur], {"axis": int(mod.start_dim)})
        elif hasattr(mod, "in_features") and getattr(mod, "weight", None) is not None and mod.weight.dim() == 2:
            emit("MatMul", [cur, const(p + "_w", mod.weight.t().contiguous())])
            if getattr(mod, "bias", None) is not None:
                emit("Add", [cur, const(p + "_b", mod.bias)])
        elif t == "Embedding":
            emit("Gather", [const(p + "_w", mod.weight), cur], {"axis": 0})
        elif t == "LayerNorm":
            emit("LayerNormalization", [cur, const(p + "_w", mod.weight), const(p + "_b", mod.bias)], {"axis": -1, "epsilon": float(mod.eps)})
        elif t == "RMSNorm":
            emit("SimplifiedLayerNormalization", [cur, const(p + "_w", mod.weight)],
                 {"axis": -1, "epsilon": float(getattr(mod, "eps", None) or 1e-6)})
        elif t in ("ReLU", "Sigmoid", "Tanh", "GELU", "SiLU", "LeakyReLU", "ELU", "Softplus", "Softmax", "LogSoftmax"):
            op = {"ReLU": "Relu", "GELU": "Gelu", "SiLU": "Swish", "LeakyReLU": "LeakyRelu", "ELU": "Elu"}.get(t, t)
            attrs = {}
            if t == "LeakyReLU":
                attrs["alpha"] = float(mod.negative_slope)
            if t == "ELU":
                attrs["alpha"] = float(mod.alpha)
            if t in ("Softmax", "LogSoftmax"):
                attrs["axis"] = int(mod.dim if mod.dim is not None else -1)
            emit(op, [cur], attrs)
        elif t in ("Dropout", "Dropout2d", "Identity"):
            continue
        else:
            raise NotImplementedError(f"export of {t}")
    g.outputs = [ValueInfo(cur, DT_FLOAT, ())]
    m = Model(g)
    if path:
        m.save(path)
    return m
