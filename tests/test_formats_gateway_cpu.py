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


def test_hierarchical_file_groups_datasets_attributes(tmp_path):
    import numpy as np
    from sneppx_alg_b200.hub.formats import HierarchicalFile
    path = str(tmp_path / "store.sxh5")
    w = torch.randn(5, 7)
    b16 = torch.randn(4, 3).bfloat16()
    with HierarchicalFile(path, "w") as f:
        f.create_group("/model/layers/0")
        f.write_dataset("/model/layers/0/weight", w)
        f.write_dataset("/model/layers/0/scale", b16)
        f.write_dataset("/stats/steps", np.arange(10, dtype=np.int64))
        f.write_dataset("/stats/empty", np.zeros((0, 4), dtype=np.float32))
        f.write_attribute("/model", "arch", {"d_model": 64, "layers": 2})
        f.write_attribute("/model/layers/0/weight", "digest", b"\x01\x02")
        assert np.array_equal(f.read_dataset("/stats/steps"), np.arange(10))      # readable before close
    with HierarchicalFile(path, "r") as f:
        assert f.list_children("/") == ["model", "stats"] and f.list_children("/model/layers/0") == ["scale", "weight"]
        assert f.dataset_exists("/model/layers/0/weight") and not f.dataset_exists("/model/layers") and f.exists("/model/layers")
        assert torch.equal(f.read_dataset("/model/layers/0/weight", as_tensor=True), w)
        assert torch.equal(f.read_dataset("/model/layers/0/scale"), b16)
        assert f.read_dataset("/stats/empty").shape == (0, 4)
        assert f.read_attribute("/model", "arch")["d_model"] == 64
        assert f.read_attribute("/model/layers/0/weight", "digest") == b"\x01\x02"
        with pytest.raises(PermissionError):
            f.write_dataset("/x", w)
        with pytest.raises(KeyError):
            f.read_dataset("/model")
    import os
    with HierarchicalFile(path, "a") as f:                                         # append + replace + repack
        f.write_dataset("/model/layers/0/weight", w * 2)
        f.write_state_dict({"head.weight": w, "head.bias": torch.zeros(7)}, root="/extra")
    grown = os.path.getsize(path)
    with HierarchicalFile(path, "a") as f:
        assert torch.equal(f.read_dataset("/model/layers/0/weight", as_tensor=True), w * 2)
        sd = f.read_state_dict("/extra")
        assert set(sd) == {"head.weight", "head.bias"} and torch.equal(sd["head.weight"], w)
        f.repack()
        assert f.read_attribute("/model", "arch")["layers"] == 2
        assert torch.equal(f.read_dataset("/model/layers/0/scale"), b16)
    assert os.path.getsize(path) < grown
    # damaged files are reported, not trusted
    raw = bytearray(open(path, "rb").read())
    open(path, "wb").write(bytes(raw[:8]) + (10 ** 12).to_bytes(8, "little") + bytes(raw[16:]))
    with pytest.raises(ValueError):
        HierarchicalFile(path, "r")
    open(path, "wb").write(b"nope")
    with pytest.raises(ValueError):
        HierarchicalFile(path, "r")


def test_raw_trainer_checkpoint_round_trip_and_damage(tmp_path):
    import struct
    from sneppx_alg_b200.checkpoint.sneppx_format import load_raw_trainer_checkpoint, save_raw_trainer_checkpoint
    p = str(tmp_path / "trainer.ckpt")
    params = [torch.randn(4, 3), torch.randn(5).bfloat16(), torch.tensor(2.5), torch.zeros(0, 2)]
    save_raw_trainer_checkpoint(p, 1234, params)
    raw = open(p, "rb").read()
    assert struct.unpack_from("<IIQQ", raw, 0) == (0x41524958, 2, 1234, 4)
    assert struct.unpack_from("<IQQQ", raw, 24) == (2, 4, 3, 12)                 # first record: ndim, shape, element count
    step, back = load_raw_trainer_checkpoint(p)
    assert step == 1234 and len(back) == 4 and all(torch.equal(b, q.float()) for b, q in zip(back, params))
    save_raw_trainer_checkpoint(p, 7, {"a": params[0]})
    assert load_raw_trainer_checkpoint(p)[1][0].shape == (4, 3)
    open(p, "wb").write(struct.pack("<IIQ", 0x41524958, 1, 99))
    assert load_raw_trainer_checkpoint(p) == (99, [])
    for bad in (raw[:10], raw[:40], b"XXXX" + raw[4:], raw[:16] + struct.pack("<Q", 1 << 50) + raw[24:],
                raw[:24] + struct.pack("<I", 9) + raw[28:], raw[:44] + struct.pack("<Q", 13) + raw[52:]):
        open(p, "wb").write(bad)
        with pytest.raises(ValueError):
            load_raw_trainer_checkpoint(p)
