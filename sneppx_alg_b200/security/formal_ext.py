"""S8 extensions around the explicit-state model checker of ``security/formal.py``.

* ``TlaSpec``: a subset of TLA+ (VARIABLES, Init, Next as a disjunction of guarded actions with primed assignments,
  ``\\in a..b`` choices, UNCHANGED, named predicates) explored into a ``FormalModel`` whose states carry the names of
  the predicates that hold, so invariants and LTL properties can be checked on it;
* ``ltl_to_string`` / ``ltl_negate`` / ``ltl_check_trace``: printing, negation and finite-trace evaluation of the
  checker's formulas;
* ``SymbolicExecutor``: path exploration of a small stack machine's byte code with symbolic integer inputs; each
  feasible path comes with its branch conditions and a concrete witness input, assertion failures with a
  counterexample, and the run reports instruction coverage;
* ``LoopProgram``: loops in a three-line notation run concretely; ``infer_invariants`` proposes bounds, monotonic
  relations and polynomial equalities (degree <= 2) that held at every loop head of every sampled run, ``verify_invariant`` checks a
  given one the same way (a bounded check, reported as such);
* ``DataFlow``: taint propagation over an assignment graph with sanitisers, to a fixed point, with DOT export;
* ``lean_export_theorem`` / ``lean_export_invariant``: Lean 4 source for a stated theorem, and for a finite-model
  invariant a self-contained file in which the state space is spelled out and the claim is closed by ``decide``.

Reference behaviour: security/formal/s8_extensions.c (function families ``tla_*``, ``ltl_*``, ``symex_*``,
``loop_invariant_*``, ``data_flow_*``, ``lean_export_*``).
"""
from __future__ import annotations

import itertools
import os
import re
import struct
from dataclasses import dataclass, field
from fractions import Fraction
from typing import Any, Dict, Iterable, List, Optional, Sequence, Set, Tuple

from .formal import CheckResult, FormalModel, parse_ltl

# ------------------------------------------------------------------------------------------------ expressions
_TOK = re.compile(r"\s*(?:(\d+)|(/\\|\\/|\\in|\.\.|<<|>>|<=|>=|=>|/=|#|==|[-+*%()<>=,~'])|([A-Za-z_][A-Za-z0-9_]*))")


class SpecError(ValueError):
    pass


def _tokenize(text: str) -> List[Tuple[str, Any]]:
    out, pos = [], 0
    text = text.replace("\\land", "/\\").replace("\\lor", "\\/").replace("\\neg", "~").replace("\\lnot", "~")
    while pos < len(text):
        if text[pos:].strip() == "":
            break
        m = _TOK.match(text, pos)
        if not m:
            raise SpecError(f"cannot read {text[pos:pos + 20]!r}")
        num, op, word = m.groups()
        out.append(("num", int(num)) if num is not None else ("op", op) if op is not None else ("id", word))
        pos = m.end()
    return out


class _Parser:
    """Precedence climbing into tuples: ("num", n) ("var", name) ("prime", name) ("not", e) ("neg", e)
    ("bin", op, a, b) ("in", e, lo, hi) ("unchanged", [names])."""

    LEVELS = (("=>",), ("\\/",), ("/\\",), ("=", "/=", "#", "<", "<=", ">", ">=", "\\in"), ("+", "-"), ("*", "%"))

    def __init__(self, tokens):
        self.t, self.i = tokens, 0

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None)

    def take(self, want=None):
        tok = self.peek()
        if want is not None and tok != want:
            raise SpecError(f"expected {want[1]!r}, found {tok[1]!r}")
        self.i += 1
        return tok

    def parse(self):
        e = self.level(0)
        if self.i != len(self.t):
            raise SpecError(f"unexpected {self.peek()[1]!r}")
        return e

    def level(self, k):
        if k == len(self.LEVELS):
            return self.unary()
        if self.LEVELS[k] in (("\\/",), ("/\\",)) and self.peek() == ("op", self.LEVELS[k][0]):
            self.take()                                       # a leading bullet, as in TLA+'s aligned lists
        left = self.level(k + 1)
        while self.peek()[0] == "op" and self.peek()[1] in self.LEVELS[k]:
            op = self.take()[1]
            if op == "\\in":
                lo = self.level(k + 1)
                self.take(("op", ".."))
                left = ("in", left, lo, self.level(k + 1))
            else:
                left = ("bin", op, left, self.level(k + 1))
        return left

    def unary(self):
        kind, v = self.peek()
        if (kind, v) == ("op", "~"):
            self.take()
            return ("not", self.unary())
        if (kind, v) == ("op", "-"):
            self.take()
            return ("neg", self.unary())
        if (kind, v) == ("op", "("):
            self.take()
            e = self.level(0)
            self.take(("op", ")"))
            return e
        if kind == "num":
            self.take()
            return ("num", v)
        if kind == "id":
            self.take()
            if v in ("TRUE", "FALSE"):
                return ("num", int(v == "TRUE"))
            if v == "UNCHANGED":
                names = []
                if self.peek() == ("op", "<<"):
                    self.take()
                    while self.peek() != ("op", ">>"):
                        names.append(self.take()[1])
                        if self.peek() == ("op", ","):
                            self.take()
                    self.take()
                else:
                    names.append(self.take()[1])
                return ("unchanged", names)
            if self.peek() == ("op", "'"):
                self.take()
                return ("prime", v)
            return ("var", v)
        raise SpecError(f"unexpected {v!r}")


def parse_expr(text: str):
    return _Parser(_tokenize(text)).parse()


def eval_expr(e, env: Dict[str, int], primed: Optional[Dict[str, int]] = None, defs: Optional[Dict[str, Any]] = None):
    k = e[0]
    if k == "num":
        return e[1]
    if k == "var":
        if e[1] in env:
            return env[e[1]]
        if defs and e[1] in defs:
            return eval_expr(defs[e[1]], env, primed, defs)
        raise SpecError(f"unknown name {e[1]!r}")
    if k == "prime":
        if primed is None or e[1] not in primed:
            raise SpecError(f"{e[1]}' is not determined here")
        return primed[e[1]]
    if k == "not":
        return int(not eval_expr(e[1], env, primed, defs))
    if k == "neg":
        return -eval_expr(e[1], env, primed, defs)
    if k == "in":
        v = eval_expr(e[1], env, primed, defs)
        return int(eval_expr(e[2], env, primed, defs) <= v <= eval_expr(e[3], env, primed, defs))
    if k == "unchanged":
        return int(primed is not None and all(primed.get(n) == env[n] for n in e[1]))
    op, a, b = e[1], e[2], e[3]
    if op == "/\\":
        return int(bool(eval_expr(a, env, primed, defs)) and bool(eval_expr(b, env, primed, defs)))
    if op == "\\/":
        return int(bool(eval_expr(a, env, primed, defs)) or bool(eval_expr(b, env, primed, defs)))
    if op == "=>":
        return int(not eval_expr(a, env, primed, defs) or bool(eval_expr(b, env, primed, defs)))
    x, y = eval_expr(a, env, primed, defs), eval_expr(b, env, primed, defs)
    if op in ("+", "-", "*"):
        return x + y if op == "+" else x - y if op == "-" else x * y
    if op == "%":
        if y == 0:
            raise SpecError("modulo by zero")
        return x % y
    return int({"=": x == y, "/=": x != y, "#": x != y, "<": x < y, "<=": x <= y, ">": x > y, ">=": x >= y}[op])


def _has_prime(e) -> bool:
    if e[0] in ("prime", "unchanged"):
        return True
    return any(isinstance(c, tuple) and _has_prime(c) for c in e[1:])


def _split(e, op: str) -> List:
    return _split(e[2], op) + _split(e[3], op) if e[0] == "bin" and e[1] == op else [e]


# ------------------------------------------------------------------------------------------------ TLA+ subset
class TlaSpec:
    """A specification over integer (and 0 / 1 boolean) variables::

        VARIABLES x, turn
        Init == x = 0 /\\ turn \\in 0..1
        Next == \\/ (x < 3 /\\ x' = x + 1 /\\ UNCHANGED turn)
                \\/ (x = 3 /\\ x' = 0 /\\ turn' = 1 - turn)
        Bounded == x <= 3
        AtTop == x = 3

    ``Init`` is a conjunction of ``v = e`` / ``v \\in a..b``; each disjunct of ``Next`` is a conjunction of guards
    (no primes), ``v' = e``, ``v' \\in a..b`` and UNCHANGED; a variable an action does not mention keeps its value.
    Every other definition without primes is a named predicate."""

    def __init__(self, text: str):
        self.variables: List[str] = []
        self.defs: Dict[str, Any] = {}
        self.error = ""
        try:
            self._parse(text)
        except SpecError as e:
            self.error = str(e)
            raise

    def _parse(self, text: str) -> None:
        text = re.sub(r"\\\*.*", "", text)
        text = re.sub(r"^-{4,}.*$|^={4,}\s*$|^\s*EXTENDS.*$", "", text, flags=re.M)
        chunks = re.split(r"^\s*(VARIABLES?\b|[A-Za-z_]\w*\s*==)", text, flags=re.M)
        for head, body in zip(chunks[1::2], chunks[2::2]):
            head = head.strip()
            if head.startswith("VARIABLE"):
                self.variables += [v.strip() for v in body.replace("\n", " ").split(",") if v.strip()]
            else:
                self.defs[head[:-2].strip()] = parse_expr(body)
        if not self.variables:
            raise SpecError("no VARIABLES declaration")
        for need in ("Init", "Next"):
            if need not in self.defs:
                raise SpecError(f"no {need} definition")
        self.predicates = {n: e for n, e in self.defs.items() if n not in ("Init", "Next") and not _has_prime(e)}

    # ---- semantics
    def initial_states(self) -> List[Tuple[int, ...]]:
        choices: Dict[str, List[int]] = {}
        guards = []
        for c in _split(self.defs["Init"], "/\\"):
            if c[0] == "bin" and c[1] == "=" and c[2][0] == "var" and c[2][1] in self.variables and c[2][1] not in choices:
                choices[c[2][1]] = [eval_expr(c[3], {}, None, None)]
            elif c[0] == "in" and c[1][0] == "var" and c[1][1] in self.variables and c[1][1] not in choices:
                choices[c[1][1]] = list(range(eval_expr(c[2], {}), eval_expr(c[3], {}) + 1))
            else:
                guards.append(c)
        missing = [v for v in self.variables if v not in choices]
        if missing:
            raise SpecError(f"Init does not fix {', '.join(missing)}")
        out = []
        for combo in itertools.product(*(choices[v] for v in self.variables)):
            env = dict(zip(self.variables, combo))
            if all(eval_expr(g, env, None, self.predicates) for g in guards):
                out.append(combo)
        return out

    def successors(self, state: Tuple[int, ...]) -> List[Tuple[Tuple[int, ...], int]]:
        """(next state, index of the action that produced it) for every enabled action and every choice in it."""
        env = dict(zip(self.variables, state))
        out = []
        for ai, action in enumerate(_split(self.defs["Next"], "\\/")):
            choices: Dict[str, List[int]] = {}
            guards, post = [], []
            for c in _split(action, "/\\"):
                if c[0] == "bin" and c[1] == "=" and c[2][0] == "prime" and not _has_prime(c[3]) and c[2][1] not in choices:
                    choices[c[2][1]] = [eval_expr(c[3], env, None, self.predicates)]
                elif c[0] == "in" and c[1][0] == "prime" and c[1][1] not in choices:
                    choices[c[1][1]] = list(range(eval_expr(c[2], env, None, self.predicates),
                                                  eval_expr(c[3], env, None, self.predicates) + 1))
                elif c[0] == "unchanged":
                    for n in c[1]:
                        choices.setdefault(n, [env[n]])
                elif _has_prime(c):
                    post.append(c)
                else:
                    guards.append(c)
            if not all(eval_expr(g, env, None, self.predicates) for g in guards):
                continue
            for v in self.variables:
                choices.setdefault(v, [env[v]])
            for combo in itertools.product(*(choices[v] for v in self.variables)):
                primed = dict(zip(self.variables, combo))
                if all(eval_expr(p, env, primed, self.predicates) for p in post):
                    out.append((combo, ai))
        return out

    def explore(self, max_states: int = 100000) -> Tuple[FormalModel, Dict[Tuple[int, ...], int]]:
        """Breadth-first exploration. Returns the model (state ids in discovery order, each labelled with the names of
        the predicates true in it) and the map from variable valuations to state ids."""
        ids: Dict[Tuple[int, ...], int] = {}
        model = FormalModel()
        frontier = []
        for s in self.initial_states():
            if s not in ids:
                ids[s] = len(ids)
                model.add_state(ids[s], self._props(s), initial=True)
                frontier.append(s)
        while frontier:
            nxt = []
            for s in frontier:
                for t, ai in self.successors(s):
                    if t not in ids:
                        if len(ids) >= max_states:
                            raise SpecError(f"more than {max_states} reachable states")
                        ids[t] = len(ids)
                        model.add_state(ids[t], self._props(t))
                        nxt.append(t)
                    model.add_transition(ids[s], ids[t], f"a{ai}")
            frontier = nxt
        return model, ids

    def _props(self, state) -> List[str]:
        env = dict(zip(self.variables, state))
        return [n for n, e in self.predicates.items() if eval_expr(e, env, None, self.predicates)]

    def check_invariant(self, name: str, max_states: int = 100000) -> Tuple[bool, Optional[List[Dict[str, int]]]]:
        """(holds, shortest trace of variable valuations to a violating state)."""
        if name not in self.predicates:
            raise SpecError(f"no predicate named {name}")
        model, ids = self.explore(max_states)
        res = model.verify_invariant(lambda s, props: name in props)
        if res.holds:
            return True, None
        back = {i: s for s, i in ids.items()}
        return False, [dict(zip(self.variables, back[i])) for i in res.counterexample]

    def check_ltl(self, formula: str, max_states: int = 100000) -> CheckResult:
        model, _ = self.explore(max_states)
        return model.check_ltl(parse_ltl(formula))

    def state_count(self, max_states: int = 100000) -> int:
        return self.explore(max_states)[0].state_count


def tla_parse_file(path: str) -> TlaSpec:
    with open(path) as f:
        return TlaSpec(f.read())


# ------------------------------------------------------------------------------------------------ LTL helpers
_UN = {"not": "!", "next": "X", "always": "G", "eventually": "F"}
_BI = {"and": "&", "or": "|", "implies": "->", "until": "U", "release": "R"}


def ltl_to_string(f) -> str:
    """Text that ``parse_ltl`` reads back to the same formula."""
    if f is True or f is False:
        return "true" if f else "false"
    if f[0] == "ap":
        return f[1]
    if f[0] in _UN:
        return f"{_UN[f[0]]} {_wrap(f[1])}"
    return f"{_wrap(f[1])} {_BI[f[0]]} {_wrap(f[2])}"


def _wrap(f) -> str:
    s = ltl_to_string(f)
    return s if f is True or f is False or f[0] == "ap" else f"({s})"


def ltl_negate(formula) -> str:
    """The negation of a formula (text or tuples), pushed one level inward where a dual exists."""
    f = parse_ltl(formula) if isinstance(formula, str) else formula
    if f is True or f is False:
        return ltl_to_string(not f)
    if f[0] == "not":
        return ltl_to_string(f[1])
    dual = {"always": "eventually", "eventually": "always", "next": "next"}
    if f[0] in dual:
        return ltl_to_string((dual[f[0]], ("not", f[1])))
    return ltl_to_string(("not", f))


def ltl_check_trace(trace: Sequence[Iterable[str]], formula, i: int = 0) -> bool:
    """Finite-trace semantics: ``trace[i]`` is the set of propositions true at step i; X is false at the last step,
    G / R range over the remaining steps."""
    f = parse_ltl(formula) if isinstance(formula, str) else formula
    n = len(trace)
    if f is True or f is False:
        return bool(f)
    op = f[0]
    if op == "ap":
        return i < n and f[1] in trace[i]
    if op == "not":
        return not ltl_check_trace(trace, f[1], i)
    if op == "and":
        return ltl_check_trace(trace, f[1], i) and ltl_check_trace(trace, f[2], i)
    if op == "or":
        return ltl_check_trace(trace, f[1], i) or ltl_check_trace(trace, f[2], i)
    if op == "implies":
        return not ltl_check_trace(trace, f[1], i) or ltl_check_trace(trace, f[2], i)
    if op == "next":
        return i + 1 < n and ltl_check_trace(trace, f[1], i + 1)
    if op == "always":
        return all(ltl_check_trace(trace, f[1], j) for j in range(i, n))
    if op == "eventually":
        return any(ltl_check_trace(trace, f[1], j) for j in range(i, n))
    if op == "until":
        for j in range(i, n):
            if ltl_check_trace(trace, f[2], j):
                return True
            if not ltl_check_trace(trace, f[1], j):
                return False
        return False
    if op == "release":
        for j in range(i, n):
            if not ltl_check_trace(trace, f[2], j):
                return False
            if ltl_check_trace(trace, f[1], j):
                return True
        return True
    raise ValueError(f"unknown operator {op!r}")


# ------------------------------------------------------------------------------------------------ symbolic execution
# A small stack machine. Every instruction is one opcode byte; PUSH carries a 4-byte signed operand, LOAD / jumps a
# 2-byte operand (input index / absolute target).
SX_PUSH, SX_LOAD, SX_ADD, SX_SUB, SX_MUL, SX_NEG, SX_DUP, SX_POP, SX_SWAP, SX_LT, SX_LE, SX_EQ, SX_NE, SX_NOT, SX_JMP, SX_JZ, \
    SX_JNZ, SX_ASSERT, SX_RET = range(1, 20)
_SX_NAMES = {v: k[3:].lower() for k, v in list(globals().items()) if k.startswith("SX_")}
_SX_WIDTH = {SX_PUSH: 5, SX_LOAD: 3, SX_JMP: 3, SX_JZ: 3, SX_JNZ: 3}


def sx_assemble(lines: Iterable[str]) -> bytes:
    """``push 3`` / ``load 0`` / ``add`` / ``jz done`` / ``done:`` ... : mnemonics with labels, to byte code."""
    names = {v: k for k, v in _SX_NAMES.items()}
    items, labels, pc = [], {}, 0
    for raw in lines:
        line = raw.split(";")[0].strip()
        if not line:
            continue
        if line.endswith(":"):
            labels[line[:-1]] = pc
            continue
        parts = line.split()
        if parts[0] not in names:
            raise SpecError(f"unknown mnemonic {parts[0]!r}")
        op = names[parts[0]]
        items.append((op, parts[1] if len(parts) > 1 else None))
        pc += _SX_WIDTH.get(op, 1)
    out = bytearray()
    for op, arg in items:
        out.append(op)
        if op == SX_PUSH:
            out += struct.pack(">i", int(arg))
        elif op in _SX_WIDTH:
            target = labels[arg] if op != SX_LOAD and arg in labels else int(arg)
            out += struct.pack(">H", target)
    return bytes(out)


def sx_run(code: bytes, inputs: Sequence[int], max_steps: int = 10000) -> Tuple[Optional[int], bool]:
    """Concrete run: (returned value or None, whether an assertion failed)."""
    stack: List[int] = []
    pc = steps = 0
    while pc < len(code):
        steps += 1
        if steps > max_steps:
            raise SpecError("step limit reached")
        op = code[pc]
        if op == SX_PUSH:
            stack.append(struct.unpack(">i", code[pc + 1:pc + 5])[0])
        elif op == SX_LOAD:
            stack.append(inputs[struct.unpack(">H", code[pc + 1:pc + 3])[0]])
        elif op in (SX_JMP, SX_JZ, SX_JNZ):
            t = struct.unpack(">H", code[pc + 1:pc + 3])[0]
            if op == SX_JMP or (stack.pop() == 0) == (op == SX_JZ):
                pc = t
                continue
        elif op == SX_ASSERT:
            if stack.pop() == 0:
                return None, True
        elif op == SX_RET:
            return (stack.pop() if stack else 0), False
        elif op == SX_NEG:
            stack.append(-stack.pop())
        elif op == SX_NOT:
            stack.append(int(stack.pop() == 0))
        elif op == SX_DUP:
            stack.append(stack[-1])
        elif op == SX_POP:
            stack.pop()
        elif op == SX_SWAP:
            stack[-1], stack[-2] = stack[-2], stack[-1]
        else:
            b, a = stack.pop(), stack.pop()
            stack.append({SX_ADD: a + b, SX_SUB: a - b, SX_MUL: a * b, SX_LT: int(a < b), SX_LE: int(a <= b),
                          SX_EQ: int(a == b), SX_NE: int(a != b)}[op])
        pc += _SX_WIDTH.get(op, 1)
    return None, False


def _sym_eval(e, inputs: Sequence[int]) -> int:
    if isinstance(e, int):
        return e
    k = e[0]
    if k == "in":
        return inputs[e[1]]
    if k == "neg":
        return -_sym_eval(e[1], inputs)
    if k == "not":
        return int(_sym_eval(e[1], inputs) == 0)
    a, b = _sym_eval(e[1], inputs), _sym_eval(e[2], inputs)
    return {"add": a + b, "sub": a - b, "mul": a * b, "lt": int(a < b), "le": int(a <= b), "eq": int(a == b), "ne": int(a != b)}[k]


def _sym_str(e) -> str:
    if isinstance(e, int):
        return str(e)
    if e[0] == "in":
        return f"x{e[1]}"
    if e[0] in ("neg", "not"):
        return ("-" if e[0] == "neg" else "!") + _sym_str(e[1])
    sym = {"add": "+", "sub": "-", "mul": "*", "lt": "<", "le": "<=", "eq": "==", "ne": "!="}[e[0]]
    return f"({_sym_str(e[1])} {sym} {_sym_str(e[2])})"


@dataclass
class SymPath:
    conditions: List[str]              # branch conditions in program order, as text over x0, x1, ...
    witness: Tuple[int, ...]           # concrete inputs that drive execution down this path
    result: Optional[str]              # symbolic return value, or None when the path ends in a failed assertion
    assertion_failed: bool = False
    pcs: List[int] = field(default_factory=list)


class SymbolicExecutor:
    """Explores every path of a program whose ``num_inputs`` inputs are unknown integers in ``[-bound, bound]``. At a
    branch on a symbolic value both sides are followed; a side is kept only if some input in the box satisfies the
    conditions collected so far (checked by search over the box: exhaustive for small boxes, boundary and random
    points otherwise), which also yields the witness. Loops unroll up to ``depth_limit`` branch decisions per path."""

    def __init__(self, num_inputs: int, bound: int = 8, depth_limit: int = 32, max_paths: int = 4096, seed: int = 0):
        self.num_inputs, self.bound, self.depth_limit, self.max_paths = num_inputs, bound, depth_limit, max_paths
        self._seed = seed
        self.reset()

    def reset(self) -> None:
        self.paths: List[SymPath] = []
        self.covered: Set[int] = set()
        self.truncated = 0
        self._code = b""

    def set_depth_limit(self, limit: int) -> None:
        self.depth_limit = int(limit)

    def _candidates(self) -> Iterable[Tuple[int, ...]]:
        b, n = self.bound, self.num_inputs
        if (2 * b + 1) ** n <= 50000:
            return itertools.product(range(-b, b + 1), repeat=n)
        import random
        rng = random.Random(self._seed)
        edge = [-b, -1, 0, 1, b]
        pts = list(itertools.islice(itertools.product(edge, repeat=n), 5000))
        return pts + [tuple(rng.randint(-b, b) for _ in range(n)) for _ in range(20000)]

    def _solve(self, conds) -> Optional[Tuple[int, ...]]:
        for cand in self._candidates():
            if all((_sym_eval(e, cand) != 0) == want for e, want in conds):
                return tuple(cand)
        return None

    def explore(self, code: bytes) -> List[SymPath]:
        self.reset()
        self._code = code
        work = [(0, [], [], [], 0)]                          # pc, stack, conditions, visited pcs, decisions
        while work:
            pc, stack, conds, pcs, depth = work.pop()
            while True:
                if pc >= len(code):
                    self._finish(conds, pcs, None, False)
                    break
                op = code[pc]
                pcs = pcs + [pc]
                nxt = pc + _SX_WIDTH.get(op, 1)
                if op == SX_PUSH:
                    stack = stack + [struct.unpack(">i", code[pc + 1:pc + 5])[0]]
                elif op == SX_LOAD:
                    stack = stack + [("in", struct.unpack(">H", code[pc + 1:pc + 3])[0])]
                elif op == SX_JMP:
                    nxt = struct.unpack(">H", code[pc + 1:pc + 3])[0]
                elif op in (SX_JZ, SX_JNZ, SX_ASSERT):
                    v, stack = stack[-1], stack[:-1]
                    target = struct.unpack(">H", code[pc + 1:pc + 3])[0] if op != SX_ASSERT else None
                    if isinstance(v, int):
                        if op == SX_ASSERT:
                            if v == 0:
                                self._finish(conds, pcs, None, True)
                                break
                        elif (v == 0) == (op == SX_JZ):
                            nxt = target
                    else:
                        if depth >= self.depth_limit or len(self.paths) + len(work) >= self.max_paths:
                            self.truncated += 1
                            break
                        # the value is non-zero on one side, zero on the other
                        nz_pc = nxt if op in (SX_JZ, SX_ASSERT) else target
                        z_pc = target if op == SX_JZ else (None if op == SX_ASSERT else nxt)
                        if self._solve(conds + [(v, False)]) is not None:
                            if z_pc is None:
                                self._finish(conds + [(v, False)], pcs, None, True)
                            else:
                                work.append((z_pc, stack, conds + [(v, False)], pcs, depth + 1))
                        if self._solve(conds + [(v, True)]) is None:
                            break
                        conds, depth, nxt = conds + [(v, True)], depth + 1, nz_pc
                elif op == SX_RET:
                    self._finish(conds, pcs, stack[-1] if stack else 0, False)
                    break
                elif op in (SX_NEG, SX_NOT):
                    v = stack[-1]
                    r = (-v if op == SX_NEG else int(v == 0)) if isinstance(v, int) else ("neg" if op == SX_NEG else "not", v)
                    stack = stack[:-1] + [r]
                elif op == SX_DUP:
                    stack = stack + [stack[-1]]
                elif op == SX_POP:
                    stack = stack[:-1]
                elif op == SX_SWAP:
                    stack = stack[:-2] + [stack[-1], stack[-2]]
                else:
                    a, b = stack[-2], stack[-1]
                    name = {SX_ADD: "add", SX_SUB: "sub", SX_MUL: "mul", SX_LT: "lt", SX_LE: "le", SX_EQ: "eq", SX_NE: "ne"}[op]
                    r = _sym_eval((name, a, b), ()) if isinstance(a, int) and isinstance(b, int) else (name, a, b)
                    stack = stack[:-2] + [r]
                pc = nxt
        return self.paths

    def _finish(self, conds, pcs, result, failed: bool) -> None:
        witness = self._solve(conds)
        if witness is None:
            return
        self.covered.update(pcs)
        text = [(_sym_str(e) if want else f"!{_sym_str(e)}") for e, want in conds]
        self.paths.append(SymPath(text, witness, None if result is None else _sym_str(result), failed, pcs))

    def path_count(self) -> int:
        return len(self.paths)

    def failures(self) -> List[SymPath]:
        return [p for p in self.paths if p.assertion_failed]

    def coverage(self) -> float:
        """Share of the program's instructions that some explored path executed."""
        starts, pc = [], 0
        while pc < len(self._code):
            starts.append(pc)
            pc += _SX_WIDTH.get(self._code[pc], 1)
        return len(self.covered & set(starts)) / len(starts) if starts else 1.0


# ------------------------------------------------------------------------------------------------ loop invariants
class LoopProgram:
    """``init; while guard: body`` over integer variables, in the expression language above::

        LoopProgram("i = 0, s = 0", "i < n", "s = s + i, i = i + 1", params=("n",))

    Assignments of the body take effect one after the other."""

    def __init__(self, init: str, guard: str, body: str, params: Sequence[str] = ()):
        self.params = tuple(params)
        self.init = [self._assign(a) for a in init.split(",") if a.strip()]
        self.guard = parse_expr(guard)
        self.body = [self._assign(a) for a in body.split(",") if a.strip()]
        self.variables = list(dict.fromkeys([v for v, _ in self.init] + [v for v, _ in self.body]))

    @staticmethod
    def _assign(text: str):
        name, _, expr = text.partition("=")
        if not name.strip().isidentifier() or not expr.strip():
            raise SpecError(f"bad assignment {text!r}")
        return name.strip(), parse_expr(expr)

    def run(self, max_iterations: int = 1000, **params) -> List[Dict[str, int]]:
        """Variable values at every arrival at the loop head (before the first iteration, after each one)."""
        env = dict(params)
        for v, e in self.init:
            env[v] = eval_expr(e, env)
        heads = [dict(env)]
        while eval_expr(self.guard, env):
            if len(heads) > max_iterations:
                raise SpecError("iteration limit reached")
            for v, e in self.body:
                env[v] = eval_expr(e, env)
            heads.append(dict(env))
        return heads


def _nullspace(rows: List[List[Fraction]]) -> List[List[Fraction]]:
    """Basis of {c : rows @ c = 0} by Gauss-Jordan elimination over the rationals."""
    m = [r[:] for r in rows]
    ncol = len(m[0]) if m else 0
    pivots, r = [], 0
    for c in range(ncol):
        p = next((i for i in range(r, len(m)) if m[i][c] != 0), None)
        if p is None:
            continue
        m[r], m[p] = m[p], m[r]
        m[r] = [x / m[r][c] for x in m[r]]
        for i in range(len(m)):
            if i != r and m[i][c] != 0:
                m[i] = [a - m[i][c] * b for a, b in zip(m[i], m[r])]
        pivots.append(c)
        r += 1
    basis = []
    for f in (c for c in range(ncol) if c not in pivots):
        v = [Fraction(0)] * ncol
        v[f] = Fraction(1)
        for i, pc in enumerate(pivots):
            v[pc] = -m[i][f]
        basis.append(v)
    return basis


def infer_invariants(loop: LoopProgram, samples: Optional[Sequence[Dict[str, int]]] = None, degree2: bool = True) -> List[str]:
    """Candidate invariants that held at every loop head of every sampled run: constant bounds per variable, order
    relations between names, and polynomial equalities of degree <= 2 over variables and parameters found as the null
    space of the matrix of observed monomial values (so ``2*s = i*i - i`` is found for the summation loop). They are
    conjectures from observation; ``verify_invariant`` re-checks one on further runs."""
    samples = samples if samples is not None else [dict(zip(loop.params, c)) for c in
                                                   itertools.product(range(0, 7), repeat=len(loop.params))]
    heads = [h for s in samples for h in loop.run(**s)]
    names = loop.variables + list(loop.params)
    out = []
    for v in loop.variables:
        lo, hi = min(h[v] for h in heads), max(h[v] for h in heads)
        if all(h[v] >= lo for h in heads) and lo == heads[0][v]:
            out.append(f"{v} >= {lo}")
    for a, b in itertools.permutations(names, 2):
        if all(h[a] <= h[b] for h in heads) and any(h[a] < h[b] for h in heads) and (a in loop.variables or b in loop.variables):
            out.append(f"{a} <= {b}")
    monos: List[Tuple[str, ...]] = [()] + [(n,) for n in names]
    if degree2:
        monos += list(itertools.combinations_with_replacement(names, 2))

    def value(h, mono):
        p = 1
        for n in mono:
            p *= h[n]
        return p

    rows = [[Fraction(value(h, m)) for m in monos] for h in heads]
    for vec in _nullspace(rows):
        den = 1
        for x in vec:
            den = den * x.denominator // _gcd(den, x.denominator)
        ints = [int(x * den) for x in vec]
        if sum(1 for x in ints if x) > 4:
            continue                                          # long combinations are rarely meaningful
        lead = next(x for x in reversed(ints) if x)
        if lead < 0:
            ints = [-x for x in ints]
        lhs = [(c, m) for c, m in zip(ints, monos) if c > 0]
        rhs = [(-c, m) for c, m in zip(ints, monos) if c < 0]
        fmt = lambda side: " + ".join(("" if c == 1 and m else f"{c}" + ("*" if m else "")) + "*".join(m) for c, m in side) or "0"  # noqa: E731
        out.append(f"{fmt(lhs)} = {fmt(rhs)}")
    return out


def _gcd(a: int, b: int) -> int:
    while b:
        a, b = b, a % b
    return abs(a) or 1


def verify_invariant(loop: LoopProgram, invariant: str, samples: Optional[Sequence[Dict[str, int]]] = None) -> Tuple[bool, Optional[Dict[str, int]]]:
    """Bounded check: (True, None) when the invariant holds at every loop head of every sampled run, else (False,
    the first violating valuation). With the default samples (every parameter in 0..12) this is exhaustive for that
    box and says nothing beyond it."""
    e = parse_expr(invariant)
    samples = samples if samples is not None else [dict(zip(loop.params, c)) for c in
                                                   itertools.product(range(0, 13), repeat=len(loop.params))]
    for s in samples:
        for h in loop.run(**s):
            if not eval_expr(e, h):
                return False, h
    return True, None


# ------------------------------------------------------------------------------------------------ taint analysis
class DataFlow:
    """Assignment graph ``dst <- srcs``. Taint starts at the marked sources and flows along edges until nothing
    changes; a variable marked as sanitiser output stops it. ``tainted_sinks`` lists the marked sinks that tainted
    data reaches, each with one path from a source."""

    def __init__(self):
        self.edges: Dict[str, Set[str]] = {}
        self.sources: Set[str] = set()
        self.sanitized: Set[str] = set()
        self.sinks: Set[str] = set()
        self.tainted: Dict[str, Optional[str]] = {}           # variable -> the variable it got the taint from

    def assign(self, dst: str, *srcs: str) -> None:
        self.edges.setdefault(dst, set()).update(srcs)
        for s in srcs:
            self.edges.setdefault(s, set())

    def taint(self, var: str) -> None:
        self.sources.add(var)
        self.edges.setdefault(var, set())

    def sanitize(self, var: str) -> None:
        self.sanitized.add(var)

    def sink(self, var: str) -> None:
        self.sinks.add(var)
        self.edges.setdefault(var, set())

    def propagate(self) -> int:
        """Runs to the fixed point; returns how many variables are tainted."""
        self.tainted = {s: None for s in self.sources if s not in self.sanitized}
        changed = True
        while changed:
            changed = False
            for dst in sorted(self.edges):
                if dst in self.tainted or dst in self.sanitized:
                    continue
                via = next((s for s in sorted(self.edges[dst]) if s in self.tainted), None)
                if via is not None:
                    self.tainted[dst] = via
                    changed = True
        return len(self.tainted)

    def taint_count(self) -> int:
        return len(self.tainted)

    def path_to(self, var: str) -> List[str]:
        out = []
        while var is not None:
            out.append(var)
            var = self.tainted.get(var)
        return out[::-1]

    def tainted_sinks(self) -> Dict[str, List[str]]:
        return {s: self.path_to(s) for s in sorted(self.sinks) if s in self.tainted}

    def clear(self) -> None:
        self.__init__()

    def export_dot(self, path: Optional[str] = None) -> str:
        lines = ["digraph dataflow {"]
        for v in sorted(self.edges):
            style = ("red" if v in self.tainted else "black", "box" if v in self.sinks else "ellipse")
            extra = ", peripheries=2" if v in self.sanitized else ""
            lines.append(f'  "{v}" [color={style[0]}, shape={style[1]}{extra}];')
        for dst in sorted(self.edges):
            lines += [f'  "{s}" -> "{dst}";' for s in sorted(self.edges[dst])]
        text = "\n".join(lines + ["}"]) + "\n"
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text


# ------------------------------------------------------------------------------------------------ Lean export
def lean_export_theorem(name: str, statement: str, proof: str = "sorry", path: Optional[str] = None, imports: Sequence[str] = ()) -> str:
    """Lean 4 source for one theorem: ``theorem <name> : <statement> := by <proof>``."""
    if not re.fullmatch(r"[A-Za-z_][A-Za-z0-9_.']*", name):
        raise ValueError(f"not a Lean identifier: {name!r}")
    body = "\n".join("  " + l for l in proof.strip().splitlines())
    text = "".join(f"import {i}\n" for i in imports) + ("\n" if imports else "") + f"theorem {name} : {statement} := by\n{body}\n"
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text


def lean_export_invariant(model: FormalModel, prop: str, name: str = "invariant_holds", path: Optional[str] = None) -> str:
    """A self-contained Lean 4 file stating that ``prop`` labels every state reachable in ``model``: the reachable
    states are listed, closure of the list under the transition relation and the labelling are decidable facts over
    finite lists, and each is closed by ``decide``. The model checker has already checked the same facts; the file
    lets an independent kernel re-check them."""
    reach = sorted(model.reachable())
    bad = [s for s in reach if prop not in model.labels[s]]
    if bad:
        raise ValueError(f"the invariant fails in state {bad[0]}; nothing to export")
    edges = sorted((a, b) for a in reach for b in model.succ[a])
    lst = lambda xs: "[" + ", ".join(str(x) for x in xs) + "]"                    # noqa: E731
    text = (f"-- generated from a {len(reach)}-state model; property: {prop}\n"
            f"def init : List Nat := {lst(sorted(model.initial))}\n"
            f"def reach : List Nat := {lst(reach)}\n"
            f"def edges : List (Nat × Nat) := [" + ", ".join(f"({a}, {b})" for a, b in edges) + "]\n"
            f"def labelled : List Nat := {lst(sorted(s for s in model.labels if prop in model.labels[s]))}\n\n"
            f"theorem {name}_init : init.all (fun s => reach.contains s) = true := by decide\n"
            f"theorem {name}_closed : edges.all (fun e => !reach.contains e.1 || reach.contains e.2) = true := by decide\n"
            f"theorem {name} : reach.all (fun s => labelled.contains s) = true := by decide\n")
    if path:
        with open(path, "w") as f:
            f.write(text)
    return text


def lean_export_all(theorems: Sequence[Tuple[str, str, str]], output_dir: str) -> List[str]:
    """One ``<name>.lean`` per (name, statement, proof); returns the paths."""
    os.makedirs(output_dir, exist_ok=True)
    paths = []
    for name, statement, proof in theorems:
        p = os.path.join(output_dir, name.replace(".", "_") + ".lean")
        lean_export_theorem(name, statement, proof, p)
        paths.append(p)
    return paths
