"""Explicit-state model checker: graph questions, invariants with counterexamples, LTL over infinite runs (Buchi
product, lasso counterexamples), bisimulation quotient, parser."""
import pytest

from sneppx_alg_b200.security.formal import FormalModel, parse_ltl


def traffic():
    m = FormalModel()
    m.add_state(0, {"red"}, initial=True)
    m.add_state(1, {"green"})
    m.add_state(2, {"yellow"})
    m.add_transition(0, 1, "go")
    m.add_transition(1, 2, "slow")
    m.add_transition(2, 0, "stop")
    return m


def test_graph_questions_and_invariants():
    m = traffic()
    m.add_state(3, {"dark"}, error=True)
    m.add_state(4, {"off"}, accepting=True)
    m.add_transition(2, 3, "power_loss")
    m.add_transition(0, 4, "shutdown")
    assert m.state_count == 5 and m.reachable() == {0, 1, 2, 3, 4}
    assert m.is_reachable(0, 3) and not m.is_reachable(3, 0)
    assert m.find_trace(0, 3) == [0, 1, 2, 3] and m.find_trace(4, 0) is None
    assert m.deadlocks() == [3] and m.deadlocks(include_accepting=True) == [3, 4]
    cyc = m.find_cycle()
    assert cyc[0] == cyc[-1] and set(cyc) == {0, 1, 2}
    bad = m.check_safety()
    assert not bad and bad.counterexample == [0, 1, 2, 3]
    assert m.verify_invariant(lambda s, lab: len(lab & {"red", "green"}) < 2)
    dot = m.to_dot()
    assert 's2 -> s3 [label="power_loss"]' in dot and "doublecircle" in dot


def test_ltl_on_infinite_runs():
    m = traffic()
    assert m.check_ltl("G F green")                       # every run sees green infinitely often
    assert m.check_ltl("G (red -> X green)")
    assert m.check_ltl("G (green -> F red)")
    assert m.check_ltl("G !(red & green)")
    assert m.check_ltl("!green U green")
    r = m.check_ltl("G !yellow")
    assert not r and r.counterexample[: r.loop_start + 1][-1] in (0, 1, 2) and 2 in r.counterexample
    assert not m.check_ltl("F G red")
    assert m.check_liveness("red")
    # a run that may stay away from the goal for ever
    m2 = FormalModel()
    m2.add_state(0, {"req"}, initial=True)
    m2.add_state(1, {"wait"})
    m2.add_state(2, {"ack"})
    m2.add_transition(0, 1)
    m2.add_transition(1, 1)          # the waiting loop
    m2.add_transition(1, 2)
    m2.add_transition(2, 0)
    r = m2.check_ltl("G (req -> F ack)")
    assert not r
    loop = r.counterexample[r.loop_start + 1:]
    assert loop and set(loop) == {1}                                    # the lasso stays in the waiting state
    assert m2.check_ltl("G (ack -> X req)") and not m2.check_liveness("ack")
    # a deadlock state stutters: F G done holds once the run is stuck there
    m3 = FormalModel()
    m3.add_state(0, initial=True)
    m3.add_state(1, {"done"})
    m3.add_transition(0, 1)
    assert m3.check_ltl("F G done") and m3.check_ltl("X done") and not m3.check_ltl("G !done")
    # release: ack must hold up to and including the first req... phrased on this model
    assert m3.check_ltl(("release", ("ap", "done"), True))


def test_until_needs_the_right_side_to_happen():
    m = FormalModel()
    m.add_state(0, {"a"}, initial=True)
    m.add_transition(0, 0)
    assert not m.check_ltl("a U b")            # a for ever, b never
    assert m.check_ltl("a R a") and m.check_ltl("G a")
    m.add_state(1, {"b"})
    m.add_transition(0, 1)
    m.add_transition(1, 1)
    assert not m.check_ltl("a U b")            # the run that loops on state 0 is still there
    assert m.check_ltl("G (b -> G b)")


def test_minimize_and_parser():
    m = FormalModel()
    m.add_state(0, {"p"}, initial=True)
    for s in (1, 2):                 # two bisimilar branches
        m.add_state(s, {"q"})
        m.add_transition(0, s)
        m.add_transition(s, 3)
    m.add_state(3, {"r"})
    m.add_transition(3, 3)
    q = m.minimize()
    assert q.state_count == 3
    assert q.check_ltl("p & X q & X X G r") and m.check_ltl("p & X q & X X G r")
    assert parse_ltl("G (req -> F ack)") == ("always", ("implies", ("ap", "req"), ("eventually", ("ap", "ack"))))
    assert parse_ltl("a U b U c") == ("until", ("ap", "a"), ("until", ("ap", "b"), ("ap", "c")))
    with pytest.raises(ValueError):
        parse_ltl("G (a ->")
