"""Weight-file dispatch (.pth / .npy / .npz / safetensors) and the AI gateway's routing rules."""
import pytest
import torch

from sneppx_alg_b200.hub import formats
from sneppx_alg_b200.utils.registry import AIGateway


def test_pth_npy_and_dispatch(tmp_path):
    sd = {"a.weight": torch.randn(3, 4), "b": torch.arange(5)}
    p = str(tmp_path / "m.pth")
    formats.save_pth(p, sd)
    back = formats.load_any(p)
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    torch.save({"epoch": 3, "state_dict": sd}, str(tmp_path / "wrapped.pt"))
    assert torch.equal(formats.load_pth(str(tmp_path / "wrapped.pt"))["a.weight"], sd["a.weight"])
    torch.save({"not": "tensors"}, str(tmp_path / "bad.pt"))
    with pytest.raises(ValueError):
        formats.load_pth(str(tmp_path / "bad.pt"))
    formats.save_npy(str(tmp_path / "x.npy"), sd["a.weight"])
    assert torch.equal(formats.load_npy(str(tmp_path / "x.npy")), sd["a.weight"])
    formats.save_safetensors(str(tmp_path / "m.safetensors"), sd)
    assert torch.equal(formats.load_any(str(tmp_path / "m.safetensors"))["b"], sd["b"])
    with pytest.raises(ValueError):
        formats.load_any(str(tmp_path / "m.xyz"))


def test_gateway_weights_fallback_and_rate_limit():
    gw = AIGateway()

    def broken(_):
        raise RuntimeError("down")

    gw.add_route("chat", "primary", lambda p: f"P:{p}", weight=3.0)
    gw.add_route("chat", "secondary", lambda p: f"S:{p}", weight=1.0)
    picks = [gw.query("chat", "x", request_id=f"r{i}")[0] for i in range(400)]
    assert 0.65 < picks.count("primary") / 400 < 0.85
    assert gw.query("chat", "x", request_id="same")[0] == gw.query("chat", "x", request_id="same")[0]
    gw2 = AIGateway()
    gw2.add_route("r", "bad", broken, weight=100.0)
    gw2.add_route("r", "good", lambda p: p * 2)
    assert gw2.query("r", 21, "id") == ("good", 42) and gw2.usage("r")["bad"]["failures"] == 1
    gw3 = AIGateway()
    gw3.add_route("r", "limited", lambda p: "L", rate_limit_per_s=2.0)
    gw3.add_route("r", "overflow", lambda p: "O", weight=1e-9)
    got = [gw3.query("r", None, "k", now=0.0)[1] for _ in range(4)]
    assert got == ["L", "L", "O", "O"] and gw3.query("r", None, "k", now=1.0)[1] == "L"
    gw4 = AIGateway()
    gw4.add_route("r", "bad", broken)
    with pytest.raises(RuntimeError, match="all providers failed"):
        gw4.query("r", 1)
    with pytest.raises(KeyError):
        gw4.query("nope", 1)
