"""S8 extensions (``security/formal_ext.py``): the TLA+ subset, LTL helpers, symbolic execution, loop invariants,
taint propagation and Lean export."""
import pytest

from sneppx_alg_b200.security import formal_ext as fx
from sneppx_alg_b200.security.formal import FormalModel, parse_ltl

COUNTER = r"""
---- MODULE Counter ----
EXTENDS Naturals
VARIABLES x, turn
\* a counter that wraps and flips a bit when it does
Init == x = 0 /\ turn \in 0..1
Next == \/ (x < 3 /\ x' = x + 1 /\ UNCHANGED turn)
        \/ (x = 3 /\ x' = 0 /\ turn' = 1 - turn)
Bounded == x <= 3
AtTop == x = 3
Small == x <= 2
====
"""

MUTEX = r"""
VARIABLES a, b, lock
Init == a = 0 /\ b = 0 /\ lock = 0
Next == \/ (a = 0 /\ lock = 0 /\ a' = 1 /\ lock' = 1 /\ UNCHANGED b)
        \/ (a = 1 /\ a' = 0 /\ lock' = 0 /\ UNCHANGED b)
        \/ (b = 0 /\ lock = 0 /\ b' = 1 /\ lock' = 1 /\ UNCHANGED a)
        \/ (b = 1 /\ b' = 0 /\ lock' = 0 /\ UNCHANGED a)
Exclusive == ~(a = 1 /\ b = 1)
InA == a = 1
InB == b = 1
"""


def test_tla_subset_explores_and_checks():
    spec = fx.TlaSpec(COUNTER)
    assert spec.variables == ["x", "turn"] and sorted(spec.predicates) == ["AtTop", "Bounded", "Small"]
    assert spec.initial_states() == [(0, 0), (0, 1)] and spec.state_count() == 8
    assert spec.successors((3, 0)) == [((0, 1), 1)] and spec.successors((1, 1)) == [((2, 1), 0)]
    assert spec.check_invariant("Bounded") == (True, None)
    ok, trace = spec.check_invariant("Small")
    assert not ok and trace == [{"x": i, "turn": 0} for i in range(4)]
    assert spec.check_ltl("G F AtTop") and not spec.check_ltl("F G AtTop") and spec.check_ltl("G (AtTop -> X !AtTop)")
    mutex = fx.TlaSpec(MUTEX)
    assert mutex.check_invariant("Exclusive")[0] and mutex.state_count() == 3
    starve = mutex.check_ltl("G F InA")                                          # no fairness: b can take every turn
    assert not starve and starve.counterexample is not None
    broken = fx.TlaSpec(MUTEX.replace("b = 0 /\\ lock = 0 /\\ b' = 1", "b = 0 /\\ b' = 1"))
    ok, trace = broken.check_invariant("Exclusive")
    assert not ok and trace[-1]["a"] == 1 and trace[-1]["b"] == 1
    choice = fx.TlaSpec("VARIABLE v\nInit == v = 0\nNext == v' \\in 0..2 /\\ v' /= v\nAny == TRUE")
    assert sorted(t for t, _ in choice.successors((0,))) == [(1,), (2,)] and choice.state_count() == 3
    for bad, msg in (("Init == x = 0\nNext == x' = x", "no VARIABLES"), ("VARIABLES x\nInit == x = 0", "no Next"),
                     ("VARIABLES x, y\nInit == x = 0\nNext == x' = x", "does not fix y"), ("VARIABLES x\nInit == x = $\nNext == x' = x", "cannot read")):
        with pytest.raises(fx.SpecError, match=msg):
            fx.TlaSpec(bad).initial_states()
    with pytest.raises(fx.SpecError, match="more than 5"):
        fx.TlaSpec("VARIABLES n\nInit == n = 0\nNext == n' = n + 1\nP == TRUE").explore(max_states=5)


def test_ltl_printing_negation_and_finite_traces():
    for text in ("G (req -> F ack)", "a U (b & !c)", "X X done", "G F live", "(a R b) | true"):
        f = parse_ltl(text)
        assert parse_ltl(fx.ltl_to_string(f)) == f
    assert fx.ltl_negate("G p") == "F (! p)" and fx.ltl_negate("!p") == "p" and fx.ltl_negate("a U b") == "! (a U b)"
    tr = [{"req"}, set(), {"ack"}, {"req"}, {"ack", "done"}]
    assert fx.ltl_check_trace(tr, "G (req -> F ack)") and not fx.ltl_check_trace(tr + [{"req"}], "G (req -> F ack)")
    assert fx.ltl_check_trace(tr, "F done") and not fx.ltl_check_trace(tr, "G !done") and fx.ltl_check_trace(tr, "!done U done")
    assert fx.ltl_check_trace(tr, "X X ack") and not fx.ltl_check_trace(tr, "X X X X X ack") and fx.ltl_check_trace(tr, "done R !done") is False
    assert fx.ltl_check_trace([{"p"}, {"p"}], "false R p") and fx.ltl_check_trace([{"p"}, {"p", "q"}, set()], "q R p")
    for f in ("G p", "p U q", "F (p & X q)"):
        for t in ([{"p"}, {"q"}], [{"p"}, {"p"}], [set()]):
            assert fx.ltl_check_trace(t, fx.ltl_negate(f)) == (not fx.ltl_check_trace(t, f))


ABS_PROGRAM = """
 load 0
 push 0
 lt            ; x0 < 0 ?
 jz nonneg
 load 0
 neg
 jmp check
nonneg:
 load 0
check:
 dup
 push 5
 ne
 assert        ; |x0| != 5
 load 1
 add
 ret
"""


def test_symbolic_execution_finds_paths_witnesses_and_failures():
    code = fx.sx_assemble(ABS_PROGRAM.splitlines())
    assert fx.sx_run(code, (-3, 10)) == (13, False) and fx.sx_run(code, (5, 0)) == (None, True)
    se = fx.SymbolicExecutor(num_inputs=2, bound=8)
    paths = se.explore(code)
    assert se.path_count() == 4 and se.coverage() == 1.0 and se.truncated == 0
    assert sorted(p.witness[0] for p in se.failures()) == [-5, 5]
    for p in paths:
        value, failed = fx.sx_run(code, p.witness)                               # every witness really takes its path
        assert failed == p.assertion_failed
        if not failed:
            assert value == abs(p.witness[0]) + p.witness[1]
    assert {p.result for p in paths if not p.assertion_failed} == {"(-x0 + x1)", "(x0 + x1)"}
    # an infeasible branch is pruned: x0 < 0 and then x0 > 3 cannot both hold
    dead = fx.sx_assemble("load 0\npush 0\nlt\njz out\npush 3\nload 0\nlt\njz out\npush 0\nassert\nout:\npush 1\nret".splitlines())
    se.explore(dead)
    assert se.failures() == [] and se.path_count() == 2 and se.coverage() < 1.0
    # a loop on a symbolic bound unrolls until the depth limit cuts it
    loop = fx.sx_assemble("push 0\ntop:\ndup\nload 0\nlt\njz done\npush 1\nadd\njmp top\ndone:\nret".splitlines())
    se2 = fx.SymbolicExecutor(1, bound=4, depth_limit=3)
    se2.explore(loop)
    assert se2.truncated >= 1 and {p.witness for p in se2.paths} >= {(-4,), (1,), (2,)}
    se2.set_depth_limit(16)
    assert len(se2.explore(loop)) == 5 and se2.truncated == 0                    # x0 <= 0, 1, 2, 3, 4
    with pytest.raises(fx.SpecError):
        fx.sx_assemble(["frobnicate"])
    with pytest.raises(fx.SpecError, match="step limit"):
        fx.sx_run(fx.sx_assemble(["top:", "jmp top"]), ())


def test_loop_invariants_inferred_and_checked():
    summation = fx.LoopProgram("i = 0, s = 0", "i < n", "s = s + i, i = i + 1", params=("n",))
    assert summation.run(n=4)[-1] == {"n": 4, "i": 4, "s": 6} and len(summation.run(n=0)) == 1
    inv = fx.infer_invariants(summation)
    assert "i >= 0" in inv and "i <= n" in inv and "i*i = i + 2*s" in inv
    assert fx.verify_invariant(summation, "2*s = i*i - i") == (True, None)
    assert fx.verify_invariant(summation, "s <= i") == (False, {"n": 4, "i": 4, "s": 6})
    mult = fx.LoopProgram("k = 0, p = 0", "k < a", "p = p + b, k = k + 1", params=("a", "b"))
    found = fx.infer_invariants(mult, samples=[{"a": a, "b": b} for a in range(5) for b in range(-2, 4)])
    assert "b*k = p" in found or "k*b = p" in found
    assert all(fx.verify_invariant(mult, c.replace("=", "=", 1))[0] for c in found if "=" in c and "<" not in c and ">" not in c)
    with pytest.raises(fx.SpecError, match="iteration limit"):
        fx.LoopProgram("i = 0", "i >= 0", "i = i + 1").run(max_iterations=50)
    with pytest.raises(fx.SpecError):
        fx.LoopProgram("i 0", "i < 1", "i = i + 1")


def test_taint_propagation_and_lean_export(tmp_path):
    df = fx.DataFlow()
    df.taint("request.body")
    df.assign("parsed", "request.body")
    df.assign("name", "parsed")
    df.assign("clean_name", "name")
    df.sanitize("clean_name")
    df.assign("sql", "name", "template")
    df.assign("safe_sql", "clean_name", "template")
    df.assign("log_line", "config")
    for s in ("sql", "safe_sql", "log_line"):
        df.sink(s)
    assert df.propagate() == 4 and df.taint_count() == 4
    assert df.tainted_sinks() == {"sql": ["request.body", "parsed", "name", "sql"]}
    dot = df.export_dot(str(tmp_path / "flow.dot"))
    assert '"sql" [color=red, shape=box];' in dot and '"clean_name" [color=black, shape=ellipse, peripheries=2];' in dot
    df.assign("a", "b")
    df.assign("b", "a")                                                          # a cycle does not stall the fixed point
    df.taint("a")
    assert df.propagate() == 6
    df.clear()
    assert df.propagate() == 0
    text = fx.lean_export_theorem("add_comm'", "∀ a b : Nat, a + b = b + a", "intro a b\nexact Nat.add_comm a b", str(tmp_path / "t.lean"))
    assert text == "theorem add_comm' : ∀ a b : Nat, a + b = b + a := by\n  intro a b\n  exact Nat.add_comm a b\n"
    with pytest.raises(ValueError):
        fx.lean_export_theorem("bad name", "True")
    model, _ = fx.TlaSpec(COUNTER).explore()
    lean = fx.lean_export_invariant(model, "Bounded", "bounded", str(tmp_path / "inv.lean"))
    assert "def reach : List Nat := [0, 1, 2, 3, 4, 5, 6, 7]" in lean and lean.count(":= by decide") == 3
    with pytest.raises(ValueError, match="fails in state"):
        fx.lean_export_invariant(model, "Small")
    paths = fx.lean_export_all([("t1", "True", "trivial"), ("ns.t2", "1 = 1", "rfl")], str(tmp_path / "lean"))
    assert [p.rsplit("/", 1)[1] for p in paths] == ["t1.lean", "ns_t2.lean"] and "theorem ns.t2 : 1 = 1" in open(paths[1]).read()
    m = FormalModel()
    m.add_state(0, ["ok"], initial=True)
    m.add_transition(0, 1)
    m.labels[1].add("ok")
    assert "def edges : List (Nat × Nat) := [(0, 1)]" in fx.lean_export_invariant(m, "ok")
