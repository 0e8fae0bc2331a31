"""Hub registry service behind the C++ HTTP front-end, exercised through its client: accounts, organisations, API
keys, private models, upload / download with checksums, search, leaderboard, persistence."""
import pytest
import torch

from sneppx_alg_b200.hub.registry_server import HubClient, serve_hub


def test_hub_registry_end_to_end(tmp_path):
    srv = serve_hub(str(tmp_path / "hub"))
    url = f"http://127.0.0.1:{srv.port}"
    try:
        alice, bob, anon = HubClient(url), HubClient(url), HubClient(url)
        alice.register("alice", "correct horse")
        bob.register("bob", "battery staple")
        with pytest.raises(RuntimeError, match="409"):
            anon.register("alice", "whatever123")
        with pytest.raises(RuntimeError, match="400"):
            anon.register("carol", "short")
        with pytest.raises(RuntimeError, match="401"):
            anon.login("alice", "wrong password")
        alice.login("alice", "correct horse")
        bob.login("bob", "battery staple")
        with pytest.raises(RuntimeError, match="401"):
            anon.create_model("alice/m")
        with pytest.raises(RuntimeError, match="403"):
            bob.create_model("alice/m")

        # a real model directory goes up and comes back bit-identical and loadable
        from sneppx_alg_b200.hub.model_hub import ModelHub
        from sneppx_alg_b200.models import create_model
        torch.manual_seed(0)
        model = create_model("llama3-tiny")
        src = ModelHub.save_pretrained(model, str(tmp_path / "src"))
        alice.create_model("alice/tiny-llama", "a tiny llama", tags=["llama", "test"])
        sent = alice.upload(src, "alice/tiny-llama", "1.0.0", metrics={"mmlu": 25.0})
        assert "config.json" in sent and len(sent) == 2
        with pytest.raises(RuntimeError, match="409"):
            alice.upload(src, "alice/tiny-llama", "1.0.0")
        loaded = anon.load("alice/tiny-llama", str(tmp_path / "cache"))
        for (k, a), (_, b) in zip(sorted(model.state_dict().items()), sorted(loaded.state_dict().items())):
            assert torch.equal(a, b), k
        assert anon.model_info("alice/tiny-llama")["downloads"] == 2

        # organisations, API keys, private models
        alice.create_org("lab")
        alice.add_member("lab", "bob")
        key = bob.create_api_key("ci")
        ci = HubClient(url, token=key)
        ci.create_model("lab/secret", private=True, tags=["llama"])
        ci.upload(src, "lab/secret", "0.1", metrics={"mmlu": 60.0})
        assert bob.list_api_keys() == ["ci"]
        assert [m["id"] for m in anon.search(tag="llama")] == ["alice/tiny-llama"]
        assert [m["id"] for m in alice.search(tag="llama")] == ["alice/tiny-llama", "lab/secret"]
        with pytest.raises(RuntimeError, match="404"):
            anon.model_info("lab/secret")
        assert anon.search(q="nothing") == [] and anon.list_models() == ["alice/tiny-llama"]
        alice.upload(src, "alice/tiny-llama", "1.1.0", metrics={"mmlu": 31.5})
        rows = anon.leaderboard("mmlu")
        assert [(r["id"], r["version"]) for r in rows] == [("alice/tiny-llama", "1.1.0"), ("alice/tiny-llama", "1.0.0")]
        bob.delete_api_key("ci")
        with pytest.raises(RuntimeError, match="401"):
            ci.list_models() and ci.create_model("lab/other")
        with pytest.raises(RuntimeError, match="403"):
            bob.delete_model("alice/tiny-llama")
    finally:
        srv.stop()

    # state survives a restart
    srv2 = serve_hub(str(tmp_path / "hub"))
    try:
        again = HubClient(f"http://127.0.0.1:{srv2.port}")
        assert again.list_models() == ["alice/tiny-llama"]
        again.login("alice", "correct horse")
        again.delete_model("alice/tiny-llama")
        assert again.list_models() == ["lab/secret"]  # alice is a member of lab: its private model is visible to her
        assert HubClient(again.url).list_models() == []
    finally:
        srv2.stop()


def test_hub_cli_against_service(tmp_path, capsys):
    import json

    from sneppx_alg_b200.cli import hub_main
    from sneppx_alg_b200.hub.model_hub import ModelHub
    from sneppx_alg_b200.models import create_model
    srv = serve_hub(str(tmp_path / "srv"))
    url, root = f"http://127.0.0.1:{srv.port}", str(tmp_path / "home")
    run = lambda *args: hub_main(["--root", root, *args])  # noqa: E731
    try:
        assert run("whoami") == 1
        assert run("register", url, "dana", "longpassword") == 0
        src = ModelHub.save_pretrained(create_model("llama3-tiny"), str(tmp_path / "m"))
        assert run("create", "dana/tiny", "--tags", "demo") == 0
        assert run("push", src, "dana/tiny", "--version", "0.3", "--metric", "ppl=12.5") == 0
        capsys.readouterr()
        assert run("info", "dana/tiny") == 0
        info = json.loads(capsys.readouterr().out)
        assert info["versions"]["0.3"]["metrics"] == {"ppl": 12.5}
        assert run("pull", "dana/tiny", str(tmp_path / "got")) == 0
        assert sorted(p.name for p in (tmp_path / "got").iterdir()) == sorted(p.name for p in (tmp_path / "m").iterdir())
        assert run("remote-search", "--tag", "demo") == 0 and run("delete", "dana/tiny") == 0 and run("logout") == 0
        assert run("serve", "--dry-run", "--data", str(tmp_path / "srv2")) == 0
    finally:
        srv.stop()


def test_module_level_hub_verbs_against_service(tmp_path):
    import sneppx
    from sneppx_alg_b200.hub.model_hub import ModelHub
    from sneppx_alg_b200.models import create_model
    hub = sneppx.hub
    srv = serve_hub(str(tmp_path / "srv"))
    try:
        HubClient(f"http://127.0.0.1:{srv.port}").register("erin", "longpassword")
        c = hub.login(f"http://127.0.0.1:{srv.port}", "erin", "longpassword")
        c.create_model("erin/m", tags=["t"])
        src = ModelHub.save_pretrained(create_model("llama3-tiny"), str(tmp_path / "m"))
        hub.upload(src, "erin/m", "1.0", metrics={"acc": 0.5})
        assert hub.list_models() == ["erin/m"] and [m["id"] for m in hub.search(tag="t")] == ["erin/m"]
        assert hub.leaderboard("acc")[0]["id"] == "erin/m"
        model = hub.load("erin/m", dest=None) if False else ModelHub.from_pretrained(hub.download("erin/m", dest=str(tmp_path / "dl")))
        assert sum(p.numel() for p in model.parameters()) > 0
    finally:
        hub.logout()
        srv.stop()


def test_client_refuses_server_supplied_paths(tmp_path, monkeypatch):
    """A registry that answers with a file name containing a path must not make the client write outside `dest`."""
    import hashlib

    from sneppx_alg_b200.hub.registry_server import HubClient
    c = HubClient.__new__(HubClient)
    evil = b"x"
    info = {"versions": {"1": {"files": {"../escape.txt": {"sha256": hashlib.sha256(evil).hexdigest()}}}}}
    monkeypatch.setattr(c, "model_info", lambda mid: info, raising=False)
    monkeypatch.setattr(c, "_call", lambda *a, **k: evil, raising=False)
    import pytest
    with pytest.raises(RuntimeError, match="unsafe file name"):
        c.download("m", str(tmp_path / "dl"))
    assert not (tmp_path / "escape.txt").exists()
