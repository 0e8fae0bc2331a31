"""Every script under ``examples/`` runs on the CPU and returns what its description promises."""
import importlib.util
import os
import sys

import pytest

EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


def _load(name):
    if EX not in sys.path:
        sys.path.insert(0, EX)                 # the examples import their helper module by its bare name
    spec = importlib.util.spec_from_file_location(name, os.path.join(EX, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod                    # spawned ranks of the distributed example import it back by name
    spec.loader.exec_module(mod)
    return mod


def test_every_example_is_listed_and_has_a_main():
    scripts = sorted(f[:-3] for f in os.listdir(EX) if f.startswith("ex_") and f.endswith(".py"))
    readme = open(os.path.join(EX, "README.md")).read()
    assert len(scripts) == 13 and all(f"`{s}.py`" in readme for s in scripts)
    for s in scripts:
        assert callable(_load(s).main)


def test_regression_classifiers_and_autoencoder(capsys):
    fit = _load("ex_01_linear_regression").main()
    assert abs(fit["slope"] - 3.0) < 0.05 and abs(fit["intercept"] + 2.0) < 0.05
    assert _load("ex_02_mlp_classifier").main(steps=300) > 0.97
    assert _load("ex_03_cnn_image_classification").main(steps=80) > 0.95
    assert _load("ex_04_text_embedding_classifier").main() == 1.0
    assert _load("ex_05_masked_autoencoder").main(steps=100) < 0.6
    assert "y = " in capsys.readouterr().out


def test_llama_algorithms_and_serving():
    r = _load("ex_06_llama_train_generate_checkpoint").main(steps=30)
    assert r["last"] < 0.3 * r["first"] and r["valid"] and r["same"]
    t = _load("ex_07_algorithm_tour").main()
    assert t["hss"] == (2, 32, 64) and t["npe"]["matches_torch"] and t["npe"]["instructions"][1] < t["npe"]["instructions"][0]
    assert t["pipeline_loss"][1] < t["pipeline_loss"][0] and t["arc"]["fgsm_shift"] > 0
    s = _load("ex_08_serving_engine_and_http").main()
    assert len(s["outputs"]) == 4 and all(len(o) == 6 for o in s["outputs"]) and s["streamed_first"] == s["outputs"][0]
    assert s["deterministic"] and s["stats"]["cached_prefix_tokens"] >= 24
    if "rest" in s:
        assert s["rest"] == {"completion_tokens": 5, "models": ["tiny"], "filtered_status": 400, "has_metrics": True}


def test_security_distributed_quantization_and_onnx():
    sec = _load("ex_09_security_tour").main()
    assert sec["ed25519"] and sec["aes_gcm"] and sec["mlkem768"] and sec["ceremony_shares_rebuild_key"] and sec["mutex_exclusive"]
    assert sec["policy"] == [True, False, False] and "went back" in sec["tuf_rollback_refused"] and sec["jailbreak_in_base64"]
    losses = _load("ex_10_distributed_zero").main()
    assert losses[-1] < 0.1 * losses[0]
    q = _load("ex_11_quantization").main()
    assert q["int8"] < q["fp8_e4m3"] < q["mxfp4"] and q["int4_gptq"] < q["int4_awq"] < q["int4_round_to_nearest"]
    o = _load("ex_12_onnx_export_and_run").main()
    assert o["problems"] == [] and o["max_error"] < 1e-3 and o["max_error_optimised"] < 1e-3 and o["max_error_qdq"] < 0.1


def test_secure_transports():
    r = _load("ex_13_secure_transports").main()
    assert r["certificate"] == {"reply": b"REGISTER RANK 0", "alpn": "sx/1", "resumed": False}
    assert r["ticket"] == {"reply": b"BACK AGAIN", "resumed": True} and r["psk"] == {"reply": b"NO CERTIFICATE NEEDED", "psk": True}
    assert "trusted root" in r["impostor_root"]
    assert r["quic"] == {"first_datagram": 1200, "lost": 1, "confirmed": True, "stream": b"gradient shard", "keys_left": ["application"]}


def test_notebooks_are_current_and_run():
    """``examples/notebooks/*.ipynb`` are what ``to_notebook.py`` makes of the scripts today, and the cells of one of
    them execute top to bottom."""
    import json
    conv = _load("to_notebook")
    scripts = sorted(f for f in os.listdir(EX) if f.startswith("ex_") and f.endswith(".py") and not f.startswith("ex_10_"))
    books = sorted(os.listdir(os.path.join(EX, "notebooks")))
    assert books == [s[:-3] + ".ipynb" for s in scripts]
    for s in scripts:
        on_disk = json.load(open(os.path.join(EX, "notebooks", s[:-3] + ".ipynb")))
        assert on_disk == conv.convert(os.path.join(EX, s)), f"{s}: run python examples/to_notebook.py --all"
        assert on_disk["nbformat"] == 4 and on_disk["cells"][0]["cell_type"] == "markdown" and on_disk["cells"][-1]["source"][0].startswith("result = main()")
    nb = json.load(open(os.path.join(EX, "notebooks", "ex_01_linear_regression.ipynb")))
    env = {"__name__": "__notebook__"}
    for cell in nb["cells"]:
        if cell["cell_type"] == "code":
            exec(compile("".join(cell["source"]), "cell", "exec"), env)
    assert abs(env["result"]["slope"] - 3.0) < 0.05
