"""S8 formal verification: an explicit-state model checker.

``FormalModel`` is a finite transition system (states with atomic propositions, labelled transitions, initial
states). It answers reachability, shortest traces, deadlocks, cycles, invariants with counterexample traces,
safety ("bad state never reached"), bisimulation minimisation, DOT export, and checks LTL properties over its
INFINITE runs: the formula is negated, put into negation normal form, translated to a generalised Buchi automaton
by the tableau construction of Gerth, Peled, Vardi and Wolper, multiplied with the model, and the product is
searched for a reachable accepting cycle (strongly connected components; every acceptance set must be met). A
found cycle is returned as a lasso counterexample (stem + loop). Finite maximal runs (deadlocks) are extended by
stuttering on the last state, the usual convention.

Formula syntax (tuples): ``("ap", name)``, ``True`` / ``False``, ``("not", f)``, ``("and", f, g)``,
``("or", f, g)``, ``("implies", f, g)``, ``("next", f)``, ``("always", f)``, ``("eventually", f)``,
``("until", f, g)``, ``("release", f, g)``. ``parse_ltl`` reads the textual form ``G (req -> F ack)``.

The reference's counterpart keeps states / transitions in fixed arrays and answers reachability, deadlock, cycle
and a string-matched "liveness" query (security/formal/model_checking.c:28-497); ``ltl_check`` in
``security/services.py`` evaluates a formula on ONE finite trace, which is a different question.
"""
from __future__ import annotations

import re
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, FrozenSet, Iterable, List, Optional, Sequence, Set, Tuple

Formula = object


# ----------------------------------------------------------------------------------------------- formulas
def _nnf(f, neg=False):
    """Negation normal form over ap / not ap / and / or / next / until / release / True / False."""
    if f is True or f is False:
        return (not f) if neg else f
    op = f[0]
    if op == "ap":
        return ("nap", f[1]) if neg else f
    if op == "nap":
        return ("ap", f[1]) if neg else f
    if op == "not":
        return _nnf(f[1], not neg)
    if op == "and":
        return ("or" if neg else "and", _nnf(f[1], neg), _nnf(f[2], neg))
    if op == "or":
        return ("and" if neg else "or", _nnf(f[1], neg), _nnf(f[2], neg))
    if op == "implies":
        return _nnf(("or", ("not", f[1]), f[2]), neg)
    if op == "next":
        return ("next", _nnf(f[1], neg))
    if op == "eventually":          # F g = true U g ; not F g = false R not g
        return ("release", False, _nnf(f[1], True)) if neg else ("until", True, _nnf(f[1], False))
    if op == "always":              # G g = false R g ; not G g = true U not g
        return ("until", True, _nnf(f[1], True)) if neg else ("release", False, _nnf(f[1], False))
    if op == "until":
        return ("release" if neg else "until", _nnf(f[1], neg), _nnf(f[2], neg))
    if op == "release":
        return ("until" if neg else "release", _nnf(f[1], neg), _nnf(f[2], neg))
    raise ValueError(f"unknown operator {op!r}")


def parse_ltl(text: str):
    """``G (req -> F ack)``, ``a U (b & !c)``, ``X X done``, ``G F live``: operators ! & | -> X F G U R, parentheses,
    ``true`` / ``false``, identifiers as atomic propositions. U and R associate to the right and bind tighter than
    & | ->."""
    toks = re.findall(r"->|[()!&|]|[A-Za-z_][A-Za-z0-9_.]*", text)
    pos = 0

    def peek():
        return toks[pos] if pos < len(toks) else None

    def take(t=None):
        nonlocal pos
        tok = peek()
        if tok is None or (t is not None and tok != t):
            raise ValueError(f"LTL parse error near token {pos} of {text!r}")
        pos += 1
        return tok

    def unary():
        t = peek()
        if t == "!":
            take()
            return ("not", unary())
        if t in ("X", "F", "G"):
            take()
            return ({"X": "next", "F": "eventually", "G": "always"}[t], unary())
        if t == "(":
            take()
            f = implies()
            take(")")
            return f
        name = take()
        if name == "true":
            return True
        if name == "false":
            return False
        return ("ap", name)

    def until():
        left = unary()
        if peek() in ("U", "R"):
            op = take()
            return ("until" if op == "U" else "release", left, until())
        return left

    def conj():
        f = until()
        while peek() == "&":
            take()
            f = ("and", f, until())
        return f

    def disj():
        f = conj()
        while peek() == "|":
            take()
            f = ("or", f, conj())
        return f

    def implies():
        f = disj()
        if peek() == "->":
            take()
            return ("implies", f, implies())
        return f

    out = implies()
    if pos != len(toks):
        raise ValueError(f"LTL parse error: trailing input in {text!r}")
    return out


# ----------------------------------------------------------------------------------------------- LTL -> generalised Buchi
@dataclass
class _Node:
    incoming: Set[int]
    new: Set
    old: Set
    nxt: Set
    id: int = 0


def _gba(formula):
    """Tableau construction (GPVW). Returns (nodes {id: (incoming ids, old formulas, next formulas)}, acceptance sets as
    lists of node ids, one per until-subformula). Node id 0 is the virtual initial node."""
    counter = [0]
    done: Dict[int, _Node] = {}

    def fresh():
        counter[0] += 1
        return counter[0]

    def expand(node: _Node):
        if not node.new:
            for other in done.values():
                if other.old == node.old and other.nxt == node.nxt:
                    other.incoming |= node.incoming
                    return
            node.id = fresh()
            done[node.id] = node
            expand(_Node({node.id}, set(node.nxt), set(), set()))
            return
        f = node.new.pop()
        if f is False:
            return
        if f is True:
            expand(node)
            return
        op = f[0]
        if op in ("ap", "nap"):
            contra = ("nap" if op == "ap" else "ap", f[1])
            if contra in node.old:
                return
            node.old.add(f)
            expand(node)
            return
        if op == "and":
            node.new |= {x for x in (f[1], f[2]) if x not in node.old}
            node.old.add(f)
            expand(node)
            return
        if op == "next":
            node.old.add(f)
            node.nxt.add(f[1])
            expand(node)
            return
        if op in ("or", "until", "release"):
            if op == "or":
                new1, next1, new2 = {f[1]}, set(), {f[2]}
            elif op == "until":         # f U g = g or (f and X(f U g))
                new1, next1, new2 = {f[1]}, {f}, {f[2]}
            else:                       # f R g = (f and g) or (g and X(f R g))
                new1, next1, new2 = {f[2]}, {f}, {f[1], f[2]}
            n1 = _Node(set(node.incoming), set(node.new) | {x for x in new1 if x not in node.old}, set(node.old) | {f},
                       set(node.nxt) | next1)
            n2 = _Node(set(node.incoming), set(node.new) | {x for x in new2 if x not in node.old}, set(node.old) | {f},
                       set(node.nxt))
            expand(n1)
            expand(n2)
            return
        raise ValueError(op)

    expand(_Node({0}, {formula}, set(), set()))
    untils = set()

    def collect(f):
        if f is True or f is False:
            return
        if f[0] == "until":
            untils.add(f)
        for x in f[1:]:
            if isinstance(x, tuple) or x is True or x is False:
                collect(x)
    collect(formula)
    accept = []
    for u in untils:      # a node is accepting for u when it does not owe u, or already delivers its right side
        accept.append({i for i, n in done.items() if u not in n.old or u[2] in n.old or u[2] is True})
    return done, accept


def _holds(old: Set, labels: FrozenSet[str]) -> bool:
    for f in old:
        if f is True or f is False:
            continue
        if f[0] == "ap" and f[1] not in labels:
            return False
        if f[0] == "nap" and f[1] in labels:
            return False
    return True


# ----------------------------------------------------------------------------------------------- model
@dataclass
class CheckResult:
    holds: bool
    counterexample: Optional[List[int]] = None        # states of the stem followed by the loop (LTL) or the path (safety)
    loop_start: Optional[int] = None                   # index in ``counterexample`` where the loop begins (LTL only)
    states_explored: int = 0

    def __bool__(self):
        return self.holds


class FormalModel:
    def __init__(self):
        self.labels: Dict[int, Set[str]] = {}
        self.succ: Dict[int, List[int]] = {}
        self.edge_label: Dict[Tuple[int, int], str] = {}
        self.initial: Set[int] = set()
        self.accepting: Set[int] = set()
        self.error: Set[int] = set()

    # ---- construction
    def add_state(self, s: int, props: Iterable[str] = (), initial: bool = False, accepting: bool = False,
                  error: bool = False) -> None:
        self.labels.setdefault(s, set()).update(props)
        self.succ.setdefault(s, [])
        if initial:
            self.initial.add(s)
        if accepting:
            self.accepting.add(s)
        if error:
            self.error.add(s)
            self.labels[s].add("error")

    def add_transition(self, a: int, b: int, label: str = "") -> None:
        for s in (a, b):
            self.add_state(s)
        if b not in self.succ[a]:
            self.succ[a].append(b)
        if label:
            self.edge_label[(a, b)] = label

    @property
    def state_count(self) -> int:
        return len(self.labels)

    def _starts(self, start=None) -> List[int]:
        if start is not None:
            return [start]
        return sorted(self.initial) if self.initial else ([min(self.labels)] if self.labels else [])

    # ---- graph questions
    def reachable(self, start: Optional[int] = None) -> Set[int]:
        seen, dq = set(), deque(self._starts(start))
        seen.update(dq)
        while dq:
            u = dq.popleft()
            for v in self.succ.get(u, ()):
                if v not in seen:
                    seen.add(v)
                    dq.append(v)
        return seen

    def is_reachable(self, a: int, b: int) -> bool:
        return b in self.reachable(a)

    def find_trace(self, a: int, b: int) -> Optional[List[int]]:
        """A shortest path a -> b (inclusive), or None."""
        prev, dq = {a: None}, deque([a])
        while dq:
            u = dq.popleft()
            if u == b:
                path = []
                while u is not None:
                    path.append(u)
                    u = prev[u]
                return path[::-1]
            for v in self.succ.get(u, ()):
                if v not in prev:
                    prev[v] = u
                    dq.append(v)
        return None

    def deadlocks(self, include_accepting: bool = False) -> List[int]:
        """Reachable states without successors (accepting states are proper ends unless asked for)."""
        return sorted(s for s in self.reachable() if not self.succ.get(s) and (include_accepting or s not in self.accepting))

    def find_cycle(self) -> Optional[List[int]]:
        """A reachable cycle as a list of states (first == last), or None."""
        color: Dict[int, int] = {}
        for root in self._starts():
            stack = [(root, iter(self.succ.get(root, ())))]
            path = [root]
            color[root] = 1
            while stack:
                u, it = stack[-1]
                for v in it:
                    if color.get(v, 0) == 0:
                        color[v] = 1
                        path.append(v)
                        stack.append((v, iter(self.succ.get(v, ()))))
                        break
                    if color[v] == 1:
                        return path[path.index(v):] + [v]
                else:
                    color[u] = 2
                    path.pop()
                    stack.pop()
        return None

    def has_cycle(self) -> bool:
        return self.find_cycle() is not None

    def verify_invariant(self, predicate: Callable[[int, Set[str]], bool]) -> CheckResult:
        """``predicate(state, labels)`` on every reachable state; the counterexample is a shortest path to a violation."""
        prev: Dict[int, Optional[int]] = {}
        dq = deque()
        for s in self._starts():
            prev[s] = None
            dq.append(s)
        n = 0
        while dq:
            u = dq.popleft()
            n += 1
            if not predicate(u, self.labels[u]):
                path = []
                while u is not None:
                    path.append(u)
                    u = prev[u]
                return CheckResult(False, path[::-1], None, n)
            for v in self.succ.get(u, ()):
                if v not in prev:
                    prev[v] = u
                    dq.append(v)
        return CheckResult(True, None, None, n)

    def check_safety(self) -> CheckResult:
        """No error state is reachable."""
        return self.verify_invariant(lambda s, _l: s not in self.error)

    # ---- LTL
    def check_ltl(self, formula, max_product_states: int = 2_000_000) -> CheckResult:
        """Does every infinite run from the initial states satisfy ``formula`` (tuple or text)?"""
        if isinstance(formula, str):
            formula = parse_ltl(formula)
        neg = _nnf(("not", formula))
        nodes, accept_sets = _gba(neg)
        by_incoming: Dict[int, List[int]] = {}
        for i, n in nodes.items():
            for p in n.incoming:
                by_incoming.setdefault(p, []).append(i)

        def msucc(s):
            nxt = self.succ.get(s, ())
            return nxt if nxt else (s,)           # stutter at a deadlock

        def frozen(s):
            return frozenset(self.labels[s])

        # product states (model state, automaton node): the node's literals must hold in the model state
        init = [(s, q) for s in self._starts() for q in by_incoming.get(0, ()) if _holds(nodes[q].old, frozen(s))]
        index: Dict[Tuple[int, int], int] = {}
        low: Dict[Tuple[int, int], int] = {}
        on_stack: Set[Tuple[int, int]] = set()
        stack: List[Tuple[int, int]] = []
        parent: Dict[Tuple[int, int], Optional[Tuple[int, int]]] = {}
        counter = [0]
        found: List[List[Tuple[int, int]]] = []

        def psucc(ps):
            s, q = ps
            for s2 in msucc(s):
                lab = frozen(s2)
                for q2 in by_incoming.get(q, ()):
                    if _holds(nodes[q2].old, lab):
                        yield (s2, q2)

        def accepting_scc(comp: List[Tuple[int, int]]) -> bool:
            if len(comp) == 1:
                ps = comp[0]
                if ps not in set(psucc(ps)):
                    return False
            qs = {q for _, q in comp}
            return all(qs & a for a in accept_sets)

        # iterative Tarjan
        for root in init:
            if root in index or found:
                continue
            parent[root] = None
            work = [(root, psucc(root))]
            index[root] = low[root] = counter[0]
            counter[0] += 1
            stack.append(root)
            on_stack.add(root)
            while work and not found:
                v, it = work[-1]
                advanced = False
                for w in it:
                    if w not in index:
                        if len(index) >= max_product_states:
                            raise MemoryError("product automaton exceeds max_product_states")
                        parent[w] = v
                        index[w] = low[w] = counter[0]
                        counter[0] += 1
                        stack.append(w)
                        on_stack.add(w)
                        work.append((w, psucc(w)))
                        advanced = True
                        break
                    if w in on_stack:
                        low[v] = min(low[v], index[w])
                if advanced:
                    continue
                work.pop()
                if work:
                    u = work[-1][0]
                    low[u] = min(low[u], low[v])
                if low[v] == index[v]:
                    comp = []
                    while True:
                        w = stack.pop()
                        on_stack.discard(w)
                        comp.append(w)
                        if w == v:
                            break
                    if accepting_scc(comp):
                        found.append(comp)
        if not found:
            return CheckResult(True, None, None, len(index))
        comp = found[0]
        cset = set(comp)
        entry = min(comp, key=lambda ps: index[ps])
        stem = []
        u = entry
        while u is not None:
            stem.append(u)
            u = parent.get(u)
        stem.reverse()

        def path_in(a, b):      # shortest path a -> b inside the component with at least one step; states after a
            prev: Dict[Tuple[int, int], Tuple[int, int]] = {}
            dq = deque()
            for w in psucc(a):
                if w in cset and w not in prev:
                    prev[w] = a
                    dq.append(w)
            while dq:
                x = dq.popleft()
                if x == b:
                    out = [x]
                    while prev[out[-1]] != a or (out[-1] == a and len(out) == 1):
                        out.append(prev[out[-1]])
                        if len(out) > len(prev) + 1:
                            break
                    return out[::-1]
                for w in psucc(x):
                    if w in cset and w not in prev:
                        prev[w] = x
                        dq.append(w)
            return []
        loop, cur = [], entry
        for a in accept_sets:             # visit one state of every acceptance set, then return to the entry
            target = next((ps for ps in comp if ps[1] in a), None)
            if target is not None and target != cur:
                seg = path_in(cur, target)
                loop += seg
                cur = target if seg else cur
        loop += path_in(cur, entry)
        states = [s for s, _ in stem] + [s for s, _ in loop]
        return CheckResult(False, states, len(stem) - 1, len(index))

    def check_liveness(self, prop: str) -> CheckResult:
        """Every run reaches a state labelled ``prop`` infinitely often (``G F prop``)."""
        return self.check_ltl(("always", ("eventually", ("ap", prop))))

    # ---- reduction / export
    def minimize(self) -> "FormalModel":
        """Quotient by bisimulation (same labels, same initial / accepting / error flags, successors in the same
        classes), by partition refinement."""
        states = sorted(self.labels)
        block = {s: (frozenset(self.labels[s]), s in self.initial, s in self.accepting, s in self.error) for s in states}
        while True:
            sig = {s: (block[s], frozenset(block[t] for t in self.succ.get(s, ()))) for s in states}
            ids = {}
            new = {s: ids.setdefault(sig[s], len(ids)) for s in states}
            if len(set(new.values())) == len(set(block.values())):
                block = new
                break
            block = new
        out = FormalModel()
        for s in states:
            out.add_state(block[s], self.labels[s] - {"error"}, s in self.initial, s in self.accepting, s in self.error)
        for s in states:
            for t in self.succ.get(s, ()):
                out.add_transition(block[s], block[t], self.edge_label.get((s, t), ""))
        return out

    def to_dot(self) -> str:
        lines = ["digraph model {", "  rankdir=LR;"]
        for s in sorted(self.labels):
            shape = "doublecircle" if s in self.accepting else "circle"
            color = ', color="red"' if s in self.error else ""
            lab = f"{s}\\n{','.join(sorted(self.labels[s]))}" if self.labels[s] else str(s)
            lines.append(f'  s{s} [label="{lab}", shape={shape}{color}];')
            if s in self.initial:
                lines.append(f'  init{s} [shape=point]; init{s} -> s{s};')
        for a in sorted(self.succ):
            for b in self.succ[a]:
                lab = self.edge_label.get((a, b), "")
                lines.append(f'  s{a} -> s{b}' + (f' [label="{lab}"];' if lab else ";"))
        lines.append("}")
        return "\n".join(lines)

    def export_dot(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.to_dot())
