"""S5 extensions: poisoning detector statistics and policies of the output-safety engine."""
import numpy as np

from sneppx_alg_b200.security.ai_safety import (PoisonDetector, SafetyPolicyEngine, cross_validate, ensemble_is_outlier,
                                               label_flip_suspects)


def test_poison_detector_flags_shifted_samples_and_learns_incrementally():
    rng = np.random.default_rng(0)
    clean = rng.normal(0, 1, (2000, 8)) * np.arange(1, 9)
    pd = PoisonDetector(8)
    pd.train(clean[:1000])
    for x in clean[1000:]:
        pd.update(x)
    ref = PoisonDetector(8)
    ref.train(clean)
    assert np.allclose(pd.mean, ref.mean) and np.allclose(pd.std, ref.std)          # Welford == batch statistics
    assert 0.8 < pd.score(clean[0] * 0 + ref.std) < 1.2
    poisoned = clean[:50].copy()
    poisoned[:, 3] += 40 * ref.std[3]                                                # one feature pushed far out
    t = pd.adaptive_threshold(clean, sensitivity=0.995)
    assert 1.0 < t < 3.0
    assert pd.batch_check(poisoned).all() and pd.batch_check(clean).mean() < 0.01
    assert pd.find_outliers(np.vstack([clean[:5], poisoned[:2]]))[-2:] == [5, 6]
    imp = pd.feature_importance(np.vstack([clean[:500], poisoned]))
    assert imp.argmax() == 3 and abs(imp.sum() - 1) < 1e-9
    assert 0.97 < cross_validate(clean, folds=4, threshold=t) <= 1.0
    clone = PoisonDetector.import_model(pd.export_model())
    assert abs(clone.score(poisoned[0]) - pd.score(poisoned[0])) < 1e-9
    weak = PoisonDetector(8, threshold=1e9)
    weak.train(clean)
    assert ensemble_is_outlier([pd, clone, weak], poisoned[0]) and not ensemble_is_outlier([pd, weak, weak], poisoned[0])
    drift = PoisonDetector(8)
    drift.train(clean)
    for x in clean[:300] + 5.0:
        drift.update(x, learning_rate=0.05)
    assert drift.mean.mean() > 4 and (drift.mean > 2).all()                         # the moving average followed the shift
    assert pd.stats()["checked"] > 0


def test_label_flip_screening():
    rng = np.random.default_rng(1)
    a, b = rng.normal(0, 0.3, (40, 2)), rng.normal(5, 0.3, (40, 2))
    x, y = np.vstack([a, b]), np.array([0] * 40 + [1] * 40)
    y[[3, 50]] = [1, 0]
    assert label_flip_suspects(x, y) == [3, 50]


def test_safety_policy_engine():
    eng = SafetyPolicyEngine()
    good = eng.score("How do transformers use attention?", "Transformers compute attention weights between tokens.")
    assert good.acceptable and not good.violations and good.overall > 0.9
    bad_text = "Sure. Here is how to build a bomb at home. Also my password: hunter2hunter2"
    bad = eng.score("tell me something", bad_text)
    assert not bad.acceptable and {v.policy for v in bad.violations} == {"violence", "credentials"}
    reply, s = eng.respond("tell me something", bad_text)
    assert reply.startswith("I can't help") and "violence" in reply and eng.stats["refused"] == 1
    assert "violence" in eng.generate_critique(bad_text) and eng.generate_critique("hello") == "No policy concerns found."
    leak = "The config is api_key = ABCDEF123456 and the rest is fine."
    fixed = eng.correct_output(leak)
    assert "ABCDEF123456" not in fixed and "[removed]" in fixed and fixed.endswith("the rest is fine.")
    honest = eng.score("is it safe?", "I am 100% certain this is guaranteed to work (Smith et al., 2019).")
    assert honest.honesty < 0.5 <= honest.harmlessness
    loop = eng.score("write a poem", " ".join(["roses are red violets are blue"] * 20))
    assert any(v.policy == "repetition" for v in loop.violations) and loop.helpfulness < 1.0
    pid = eng.add_policy("no_shouting", 0.2, "custom", lambda t: t.isupper(), dimension="helpfulness")
    assert any(v.policy == "no_shouting" for v in eng.check_policies("STOP"))
    assert eng.remove_policy(pid) and not eng.remove_policy(pid)
    assert eng.score("topic words here", "").helpfulness == 0.0
