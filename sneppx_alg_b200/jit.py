"""``jit``: a tracing JIT (trace -> graph IR -> passes -> replay / CUDA-graph capture) and the function transforms
grad / vmap / jacobian / hessian (the reference's ``interface_bindings/jit.py``, ``graph_compiler.py`` and
``graph_optimizer.py``).

``trace(fn, *example_inputs)`` runs ``fn`` once on the example inputs under a ``TorchFunctionMode`` that records every
torch call with a tensor argument into a ``TraceGraph`` (a tape of nodes: callable, argument tree with references to
earlier values, constants held by reference so that parameter updates stay visible). Python control flow is frozen
at trace time, as in any tracing JIT; a ``TracedFunction`` therefore keys its traces by the shapes and dtypes of its
inputs and retraces on a new signature. Passes: dead-code elimination, common-subexpression elimination,
linear + bias + activation -> one GEMM launch with a fused epilogue (``ops.linear(act=)``), optional constant folding.
Replay executes the tape without re-running the Python of ``fn``; on CUDA inputs the replay can be captured into a
CUDA graph (``cuda_graph=True``), which removes launch overhead from launch-bound loops.
The transforms are ``torch.func`` and compose with traced functions (a replay is ordinary torch calls)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import func as _func
from torch.overrides import TorchFunctionMode
from torch.utils import _pytree as pytree

grad = _func.grad
value_and_grad = _func.grad_and_value
vmap = _func.vmap
jacobian = _func.jacrev
jacfwd = _func.jacfwd
hessian = _func.hessian
vjp, jvp = _func.vjp, _func.jvp


# ----------------------------------------------------------------------------- IR
@dataclass(frozen=True)
class Ref:
    """Leaf ``leaf`` of the flattened output of node ``node`` (node -1: the traced function's inputs)."""
    node: int
    leaf: int = 0


@dataclass(frozen=True)
class Const:
    index: int


@dataclass
class Node:
    target: Callable
    args: Any
    kwargs: Dict[str, Any]
    n_leaves: int = 1
    pure: bool = True
    name: str = ""

    def refs(self) -> List[Ref]:
        return [a for a in pytree.tree_leaves((self.args, self.kwargs)) if isinstance(a, Ref)]


@dataclass
class TraceGraph:
    n_inputs: int = 0
    nodes: List[Node] = field(default_factory=list)
    consts: List[torch.Tensor] = field(default_factory=list)
    outputs: Any = None            # pytree of Ref / Const / python values
    out_spec: Any = None

    def users(self) -> Dict[Tuple[int, int], int]:
        use: Dict[Tuple[int, int], int] = {}
        for n in self.nodes:
            for r in n.refs():
                use[(r.node, r.leaf)] = use.get((r.node, r.leaf), 0) + 1
        for r in pytree.tree_leaves(self.outputs):
            if isinstance(r, Ref):
                use[(r.node, r.leaf)] = use.get((r.node, r.leaf), 0) + 1
        return use

    def code(self) -> str:
        """Readable listing of the tape."""
        def show(a):
            if isinstance(a, Ref):
                return f"in{a.leaf}" if a.node < 0 else (f"v{a.node}" + (f"[{a.leaf}]" if a.leaf else ""))
            if isinstance(a, Const):
                t = self.consts[a.index]
                return f"const{a.index}<{tuple(t.shape)}>"
            return repr(a)
        lines = [f"graph({', '.join(f'in{i}' for i in range(self.n_inputs))}):"]
        for i, n in enumerate(self.nodes):
            args = [show(a) for a in pytree.tree_leaves(n.args)] + [f"{k}={show(v)}" for k, v in n.kwargs.items()
                                                                      if not isinstance(v, (list, tuple, dict))]
            lines.append(f"  v{i} = {n.name or getattr(n.target, '__name__', str(n.target))}({', '.join(args)})")
        lines.append("  return " + ", ".join(show(a) for a in pytree.tree_leaves(self.outputs)))
        return "\n".join(lines)


def _is_impure(func, kwargs) -> bool:
    name = getattr(func, "__name__", "")
    return (name.endswith("_") and not name.endswith("__")) or name in ("__setitem__", "copy_", "__set__") or \
        (kwargs or {}).get("out") is not None or name.startswith("__i") and name.endswith("__")


_RANDOM = {"rand", "randn", "randint", "rand_like", "randn_like", "dropout", "bernoulli", "multinomial", "normal", "randperm"}


class _Recorder(TorchFunctionMode):
    def __init__(self, graph: TraceGraph, inputs: List[torch.Tensor]):
        super().__init__()
        self.g = graph
        self.where: Dict[int, Ref] = {}
        self.keep: List[torch.Tensor] = []          # ids stay unique while these are alive
        self.const_index: Dict[int, int] = {}
        for i, t in enumerate(inputs):
            self.where[id(t)] = Ref(-1, i)
            self.keep.append(t)

    def _encode(self, a):
        if isinstance(a, torch.Tensor):
            r = self.where.get(id(a))
            if r is not None:
                return r
            k = self.const_index.get(id(a))
            if k is None:
                k = len(self.g.consts)
                self.g.consts.append(a)
                self.const_index[id(a)] = k
                self.keep.append(a)
            return Const(k)
        return a

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        out = func(*args, **kwargs)
        flat_in = pytree.tree_leaves((args, kwargs))
        # calls on closed-over tensors only are recorded too (they must follow later updates of those tensors;
        # ``freeze`` folds them); calls without any tensor argument are constants of this trace
        touched = any(isinstance(a, torch.Tensor) for a in flat_in)
        name = getattr(func, "__name__", "")
        leaves = [o for o in pytree.tree_leaves(out) if isinstance(o, torch.Tensor)]
        impure = _is_impure(func, kwargs)
        if not (touched or name in _RANDOM) or (not leaves and not impure):
            return out          # shape queries, tensor creation from python values: constants of this trace
        enc_args, enc_kwargs = pytree.tree_map(self._encode, (args, kwargs))
        flat_out = pytree.tree_leaves(out)
        node = Node(func, enc_args, enc_kwargs, len(flat_out), not (impure or name in _RANDOM), name)
        self.g.nodes.append(node)
        idx = len(self.g.nodes) - 1
        for k, o in enumerate(flat_out):
            if isinstance(o, torch.Tensor):
                self.where[id(o)] = Ref(idx, k)
                self.keep.append(o)
        return out


def trace_graph(fn: Callable, *example_inputs) -> TraceGraph:
    """Runs ``fn`` on the example inputs and returns the recorded tape (no passes applied)."""
    flat, _ = pytree.tree_flatten(example_inputs)
    tensors = [t for t in flat if isinstance(t, torch.Tensor)]
    g = TraceGraph(n_inputs=len(tensors))
    rec = _Recorder(g, tensors)
    with rec:
        out = fn(*example_inputs)
    leaves, spec = pytree.tree_flatten(out)
    g.outputs = [rec._encode(o) if isinstance(o, torch.Tensor) else o for o in leaves]
    g.out_spec = spec
    return g


# ----------------------------------------------------------------------------- passes
def eliminate_dead_code(g: TraceGraph) -> int:
    """Drops pure nodes none of whose results reach an output or an impure node."""
    live = set()
    work = [r.node for r in pytree.tree_leaves(g.outputs) if isinstance(r, Ref)]
    work += [i for i, n in enumerate(g.nodes) if not n.pure]
    while work:
        i = work.pop()
        if i < 0 or i in live:
            continue
        live.add(i)
        work += [r.node for r in g.nodes[i].refs()]
    return _compact(g, [i in live for i in range(len(g.nodes))])


def _compact(g: TraceGraph, keep: List[bool], forward: Optional[Dict[int, int]] = None) -> int:
    """Removes the nodes with keep[i] False; ``forward`` maps a removed node to the kept node that replaces it."""
    forward = forward or {}
    new_index, k = {}, 0
    for i, kp in enumerate(keep):
        if kp:
            new_index[i] = k
            k += 1

    def fix(a):
        if isinstance(a, Ref) and a.node >= 0:
            j = a.node
            while j in forward:
                j = forward[j]
            return Ref(new_index[j], a.leaf)
        return a
    nodes = []
    for i, n in enumerate(g.nodes):
        if keep[i]:
            n.args, n.kwargs = pytree.tree_map(fix, (n.args, n.kwargs))
            nodes.append(n)
    removed = len(g.nodes) - len(nodes)
    g.nodes = nodes
    g.outputs = [fix(o) for o in g.outputs]
    return removed


def eliminate_common_subexpressions(g: TraceGraph) -> int:
    """Two pure nodes with the same callable and the same encoded arguments compute the same value. Skipped when the
    tape has in-place nodes (an argument's value may differ between the two call sites)."""
    if any(not n.pure for n in g.nodes):
        return 0
    seen: Dict[Any, int] = {}
    forward: Dict[int, int] = {}
    keep = [True] * len(g.nodes)

    def canon(a):
        if isinstance(a, Ref) and a.node in forward:
            return Ref(forward[a.node], a.leaf)
        return a
    for i, n in enumerate(g.nodes):
        flat, spec = pytree.tree_flatten((n.args, n.kwargs))
        try:
            key = (n.target, str(spec), tuple(canon(a) if isinstance(a, (Ref, Const)) else (type(a).__name__, repr(a)) for a in flat))
            hash(key)
        except TypeError:
            continue
        j = seen.get(key)
        if j is None:
            seen[key] = i
        else:
            forward[i], keep[i] = j, False
    return _compact(g, keep, forward)


_ACTS = {"relu": "relu", "gelu": "gelu", "silu": "silu"}


def _fused_linear(x, w, b=None, act=None):
    from .ops.gemm import linear
    return linear(x, w, b, act)


def fuse_linear_activation(g: TraceGraph) -> int:
    """``F.linear(x, w, b)`` whose only user is relu / gelu (tanh form) / silu becomes one call of the GEMM with a fused
    epilogue (one launch on the GPU instead of two, and no round trip of the pre-activation through memory)."""
    use = g.users()
    fused = 0
    keep = [True] * len(g.nodes)
    forward: Dict[int, int] = {}
    for i, n in enumerate(g.nodes):
        act = _ACTS.get(n.name)
        if act is None or not n.pure:
            continue
        flat = pytree.tree_leaves(n.args)
        if not flat or not isinstance(flat[0], Ref) or flat[0].node < 0:
            continue
        if act == "gelu" and n.kwargs.get("approximate", "none") != "tanh":
            continue            # the epilogue implements the tanh form
        p = g.nodes[flat[0].node]
        if p.target is not F.linear or use.get((flat[0].node, 0), 0) != 1 or not keep[flat[0].node]:
            continue
        pa = list(p.args) + [p.kwargs.get("bias")] if len(p.args) == 2 else list(p.args)
        g.nodes[i] = Node(_fused_linear, (pa[0], pa[1], pa[2] if len(pa) > 2 else None, act), {}, 1, True, f"linear_{act}")
        keep[flat[0].node] = False
        fused += 1
    if fused:
        _compact(g, keep, forward)
    return fused


def fold_constants(g: TraceGraph) -> int:
    """Evaluates pure nodes whose inputs are all constants NOW and stores the result as a constant. Only for frozen
    weights: later changes of those tensors are no longer seen."""
    folded = 0
    value: Dict[int, Any] = {}
    keep = [True] * len(g.nodes)

    def resolve(a):
        if isinstance(a, Const):
            return g.consts[a.index]
        if isinstance(a, Ref):
            return value[a.node][a.leaf]
        return a
    for i, n in enumerate(g.nodes):
        if n.pure and n.n_leaves == 1 and all(r.node in value for r in n.refs()) and all(r.node >= 0 for r in n.refs()) and \
                (n.refs() or any(isinstance(a, Const) for a in pytree.tree_leaves((n.args, n.kwargs)))):
            args, kwargs = pytree.tree_map(resolve, (n.args, n.kwargs))
            with torch.no_grad():
                value[i] = pytree.tree_leaves(n.target(*args, **kwargs))
    if not value:
        return 0
    subst: Dict[int, Const] = {}
    for i, leaves in value.items():
        g.consts.append(leaves[0])
        subst[i] = Const(len(g.consts) - 1)
        keep[i] = False
        folded += 1

    def fix(a):
        return subst[a.node] if isinstance(a, Ref) and a.node in subst else a
    for n in g.nodes:
        n.args, n.kwargs = pytree.tree_map(fix, (n.args, n.kwargs))
    g.outputs = [fix(o) for o in g.outputs]
    _compact(g, keep)
    return folded


def optimize(g: TraceGraph, freeze: bool = False) -> Dict[str, int]:
    stats = {"cse": eliminate_common_subexpressions(g), "fused_linear": fuse_linear_activation(g)}
    if freeze:
        stats["folded"] = fold_constants(g)
    stats["dead"] = eliminate_dead_code(g)
    return stats


# ----------------------------------------------------------------------------- replay
def run_graph(g: TraceGraph, inputs: List[torch.Tensor]):
    """Executes the tape on new inputs (same number, shapes and dtypes as the example inputs of the trace)."""
    env: List[Any] = [None] * len(g.nodes)

    def resolve(a):
        if isinstance(a, Ref):
            return inputs[a.leaf] if a.node < 0 else env[a.node][a.leaf]
        if isinstance(a, Const):
            return g.consts[a.index]
        return a
    for i, n in enumerate(g.nodes):
        args, kwargs = pytree.tree_map(resolve, (n.args, n.kwargs))
        env[i] = pytree.tree_leaves(n.target(*args, **kwargs)) if n.n_leaves != 1 else [n.target(*args, **kwargs)]
        if n.n_leaves == 1 and not isinstance(env[i][0], torch.Tensor):
            env[i] = pytree.tree_leaves(env[i][0]) or env[i]
    return pytree.tree_unflatten([resolve(o) for o in g.outputs], g.out_spec)


class GraphedCallable:
    """A function captured once into a CUDA graph.  Inputs are copied into the captured static buffers before each
    replay; outputs alias the captured output buffers (clone them to keep a result across calls)."""

    def __init__(self, fn, example_inputs, warmup=3, pool=None):
        assert all(t.is_cuda for t in example_inputs), "CUDA graph capture needs CUDA tensors"
        self.static_in = [t.clone() for t in example_inputs]
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(warmup):
                fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(s)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, pool=pool), torch.no_grad():
            self.static_out = fn(*self.static_in)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_in, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        self.graph.replay()
        return self.static_out


class TracedFunction:
    """``fn`` compiled per input signature. The first call with a new (shape, dtype, device) signature traces and
    optimises; later calls replay the tape (or the CUDA graph captured from it)."""

    def __init__(self, fn: Callable, optimize_graph: bool = True, freeze: bool = False, cuda_graph: bool = False):
        self.fn, self.optimize_graph, self.freeze, self.cuda_graph = fn, optimize_graph, freeze, cuda_graph
        self.cache: Dict[Any, Tuple[TraceGraph, Optional[GraphedCallable], Dict[str, int]]] = {}
        self.traces = 0

    @staticmethod
    def _signature(tensors, others):
        return (tuple((tuple(t.shape), t.dtype, t.device.type, t.requires_grad) for t in tensors), repr(others))

    def _split(self, inputs):
        flat, spec = pytree.tree_flatten(inputs)
        tensors = [t for t in flat if isinstance(t, torch.Tensor)]
        others = [a for a in flat if not isinstance(a, torch.Tensor)]
        return tensors, others, spec

    def graph_for(self, *inputs) -> TraceGraph:
        tensors, others, _ = self._split(inputs)
        key = self._signature(tensors, others)
        if key not in self.cache:
            g = trace_graph(self.fn, *inputs)
            stats = optimize(g, self.freeze) if self.optimize_graph else {}
            captured = None
            if self.cuda_graph and tensors and all(t.is_cuda for t in tensors) and not torch.is_grad_enabled():
                captured = GraphedCallable(lambda *ts: run_graph(g, list(ts)), tensors)
            self.cache[key] = (g, captured, stats)
            self.traces += 1
        return self.cache[key][0]

    def __call__(self, *inputs):
        tensors, others, _ = self._split(inputs)
        g = self.graph_for(*inputs)
        captured = self.cache[self._signature(tensors, others)][1]
        if captured is not None and not torch.is_grad_enabled():
            return captured(*tensors)
        return run_graph(g, tensors)

    def code(self, *inputs) -> str:
        return self.graph_for(*inputs).code()

    def stats(self, *inputs) -> Dict[str, int]:
        self.graph_for(*inputs)
        tensors, others, _ = self._split(inputs)
        return dict(self.cache[self._signature(tensors, others)][2])


def trace(fn, *example_inputs, optimize_graph: bool = True, freeze: bool = False, cuda_graph: Optional[bool] = None, warmup=3):
    """Compiles ``fn`` by tracing. With example inputs the first trace happens now. ``cuda_graph``: capture the replay
    into a CUDA graph for CUDA inputs under ``torch.no_grad`` (default: on when the example inputs are CUDA tensors)."""
    on_cuda = bool(example_inputs) and all(torch.is_tensor(t) and t.is_cuda for t in example_inputs)
    tf = TracedFunction(fn, optimize_graph, freeze, on_cuda if cuda_graph is None else cuda_graph)
    if example_inputs:
        with torch.no_grad() if on_cuda else torch.enable_grad():
            tf.graph_for(*example_inputs)
    return tf


def jit(fn=None, **kw):
    """Decorator form: ``@jit`` or ``@jit(freeze=True)``; tracing happens at the first call."""
    if fn is None:
        return lambda f: TracedFunction(f, **kw)
    return TracedFunction(fn, **kw)
