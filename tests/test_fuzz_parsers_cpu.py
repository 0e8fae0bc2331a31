"""Malformed input never crashes a parser: random and mutated byte strings through the native codecs (WebSocket, MQTT,
compression streams, checkpoint reader, tokenizer, edge model loader) and the Python ones (safetensors, hub container,
ONNX). Each must return normally or raise a Python exception. Worth running against the sanitizer build of the host
library (``_build.build_host_sanitized``)."""
import os
import random
import struct

import numpy as np
import pytest
import torch

from sneppx_alg_b200.utils import mm, net

CLEAN = (ValueError, KeyError, IndexError, OSError, RuntimeError, EOFError, OverflowError, UnicodeDecodeError, AssertionError,
         TypeError, BufferError, MemoryError, struct.error)


def _mutations(seed_bytes, rng, n):
    for _ in range(n):
        b = bytearray(seed_bytes)
        for _ in range(rng.randint(1, 6)):
            op = rng.randint(0, 3)
            if op == 0 and b:
                b[rng.randrange(len(b))] = rng.randrange(256)
            elif op == 1 and b:
                del b[rng.randrange(len(b)):rng.randrange(len(b)) + rng.randint(1, 8)]
            elif op == 2:
                at = rng.randrange(len(b) + 1)
                b[at:at] = bytes(rng.randrange(256) for _ in range(rng.randint(1, 8)))
            elif b:
                b = b[: rng.randrange(len(b))]
        yield bytes(b)
    for _ in range(n // 4):
        yield bytes(rng.randrange(256) for _ in range(rng.randint(0, 64)))


def _survives(fn, data):
    try:
        fn(data)
    except CLEAN:
        pass


def test_native_wire_codecs_survive_garbage():
    rng = random.Random(1)
    ws = net.ws_encode(b"payload" * 30, opcode=2, mask_key=0x01020304)
    for d in _mutations(ws, rng, 300):
        _survives(net.ws_decode, d)
    pkt = net.mqtt_publish("a/b/c", b"x" * 40, qos=1, packet_id=7)
    for d in _mutations(pkt, rng, 300):
        _survives(net.mqtt_parse, d)
    x = np.random.default_rng(0).standard_normal(200).astype(np.float32)
    for codec in ("bfp8", "bfp4", "sparse", "none"):
        s = mm.compress(x, codec, threshold=0.5)
        for d in _mutations(s, rng, 150):
            _survives(lambda b: mm.decompress(b, 200), d)


def test_checkpoint_and_weight_file_readers_survive_garbage(tmp_path):
    from sneppx_alg_b200.checkpoint.sneppx_format import load_tensors, save_tensors, validate_checkpoint
    from sneppx_alg_b200.hub import formats
    rng = random.Random(2)
    good = tmp_path / "ok.sneppx"
    save_tensors(str(good), {"w": torch.randn(4, 5), "b": torch.arange(3).float()}, {"step": 7})
    seeds = {"sneppx": good.read_bytes()}
    formats.save_safetensors(str(tmp_path / "ok.safetensors"), {"w": torch.randn(2, 3)})
    seeds["safetensors"] = (tmp_path / "ok.safetensors").read_bytes()
    formats.save_hub_container(str(tmp_path / "ok.hub"), {"w": torch.randn(2, 3)}, {"name": "m"})
    seeds["hub"] = (tmp_path / "ok.hub").read_bytes()
    loaders = {"sneppx": lambda p: (validate_checkpoint(p), load_tensors(p)), "safetensors": formats.load_safetensors,
               "hub": formats.load_hub_container}
    for kind, seed in seeds.items():
        for i, d in enumerate(_mutations(seed, rng, 120)):
            p = tmp_path / f"bad_{kind}.bin"
            p.write_bytes(d)
            _survives(loaders[kind], str(p))


def test_tokenizer_edge_and_onnx_loaders_survive_garbage(tmp_path):
    from sneppx_alg_b200.onnx import toolkit
    from sneppx_alg_b200.utils.host import BPETokenizer, EdgeModel, write_edge_model
    rng = random.Random(3)
    tok = BPETokenizer()
    tok.train("the quick brown fox jumps over the lazy dog " * 20, 300)
    tp = tmp_path / "tok.bin"
    tok.save(str(tp))
    for d in _mutations(tp.read_bytes(), rng, 120):
        p = tmp_path / "bad_tok.bin"
        p.write_bytes(d)
        _survives(lambda q: BPETokenizer().load(q).encode("hello fox"), str(p))
    ep = tmp_path / "m.edge"
    write_edge_model(str(ep), [("matmul", np.ones((4, 3), np.float32)), ("bias", np.zeros(3, np.float32)), ("relu",)])
    for d in _mutations(ep.read_bytes(), rng, 120):
        p = tmp_path / "bad.edge"
        p.write_bytes(d)
        _survives(lambda q: EdgeModel(q).run(np.ones((2, 4), np.float32), max_width=64), str(p))
    lin = torch.nn.Linear(4, 3)
    model = toolkit.export_module(lin, torch.randn(2, 4))
    blob = model.serialize() if hasattr(model, "serialize") else model.to_bytes()
    for d in _mutations(blob, rng, 200):
        _survives(lambda b: toolkit.check_model(toolkit.Model.parse(b)), d)


def test_http_front_end_survives_malformed_requests():
    """Raw garbage, truncated headers, absurd or non-numeric Content-Length, binary paths and half-open connections must
    not take the C++ server down: a well-formed request still gets its answer afterwards."""
    import socket
    import urllib.request

    from sneppx_alg_b200.serving.native_http import NativeHttpServer
    srv = NativeHttpServer(max_body=4096)

    @srv.route("POST", "/echo/{x}")
    def echo(p, b):
        return {"x": p["x"], "n": len(b)}

    port = srv.start(workers=2)
    rng = random.Random(7)
    payloads = [b"", b"\r\n\r\n", b"GET", b"GET / HTTP/1.1\r\n", b"POST /echo/a HTTP/1.1\r\nContent-Length: 99999999999999999999\r\n\r\n",
                b"POST /echo/a HTTP/1.1\r\nContent-Length: -5\r\n\r\nabc", b"POST /echo/a HTTP/1.1\r\nContent-Length: abc\r\n\r\n",
                b"POST /echo/a HTTP/1.1\r\nContent-Length: 100\r\n\r\nshort", b"\x00\xff" * 500, b"GET /" + b"A" * 70000 + b" HTTP/1.1\r\n\r\n",
                b"POST /echo/%00%ff\"\\ HTTP/1.1\r\nContent-Length: 1\r\n\r\nx", b"GET /metrics/native HTTP/9.9\r\n" + b"X: y\r\n" * 2000 + b"\r\n"]
    payloads += [bytes(rng.randrange(256) for _ in range(rng.randint(1, 300))) for _ in range(40)]
    try:
        for p in payloads:
            s = socket.create_connection(("127.0.0.1", port), timeout=5)
            try:
                s.sendall(p)
                s.shutdown(socket.SHUT_WR)
                s.settimeout(8)
                while s.recv(4096):
                    pass
            except OSError:
                pass
            finally:
                s.close()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/echo/ok", data=b"12345", method="POST")
        assert urllib.request.urlopen(req, timeout=10).read() == b'{"x": "ok", "n": 5}'
    finally:
        srv.stop()


def test_gguf_and_hierarchical_store_survive_garbage(tmp_path):
    from sneppx_alg_b200.hub.formats import HierarchicalFile
    from sneppx_alg_b200.hub.model_card import ModelCard, load_gguf, save_gguf
    rng = random.Random(11)
    good = str(tmp_path / "g.gguf")
    save_gguf(good, {"a.weight": torch.randn(4, 32), "b": torch.randn(8).half()}, {"general.name": "x", "list": [1, 2, 3]})
    seed = open(good, "rb").read()
    p = str(tmp_path / "m.gguf")

    def gguf(d):
        open(p, "wb").write(d)
        for t in load_gguf(p)[0].values():
            t.float().sum()
    for d in _mutations(seed, rng, 400):
        _survives(gguf, d)

    hgood = str(tmp_path / "h.sxh5")
    with HierarchicalFile(hgood, "w") as f:
        f.write_dataset("/g/w", torch.randn(6, 5))
        f.write_attribute("/g", "k", {"a": 1})
    hseed = open(hgood, "rb").read()
    hp = str(tmp_path / "m.sxh5")

    def hier(d):
        open(hp, "wb").write(d)
        with HierarchicalFile(hp, "r") as f:
            for path, e in list(f.index.items()):
                if isinstance(e, dict) and e.get("kind") == "dataset":
                    np.asarray(f.read_dataset(path)).sum()
            f.list_children("/")
    for d in _mutations(hseed, rng, 400):
        _survives(hier, d)

    card = ModelCard(name="n", version="1", architecture="a").to_json().encode()
    for d in _mutations(card, rng, 300):
        _survives(lambda b: ModelCard.from_json(b.decode("utf-8", "replace")).validate(), d)


def test_post_quantum_verifiers_reject_garbage():
    from sneppx_alg_b200.security import crypto
    rng = random.Random(12)
    pk, sk = crypto.mldsa_keygen(44, seed=bytes(32))
    sig = crypto.mldsa_sign(sk, b"m", 44, deterministic=True)
    for d in _mutations(sig, rng, 60):
        assert not crypto.mldsa_verify(pk, b"m", d, 44) or d == sig
    for _ in range(40):
        junk = bytes(rng.randrange(256) for _ in range(len(sig)))
        assert not crypto.mldsa_verify(pk, b"m", junk, 44)
        assert not crypto.mldsa_verify(bytes(rng.randrange(256) for _ in range(len(pk))), b"m", sig, 44)
    ek, dk = crypto.mlkem_keygen(512, seed=bytes(64))
    _, n_dk, n_ct = crypto.mlkem_sizes(512)
    for _ in range(40):
        assert len(crypto.mlkem_decaps(dk, bytes(rng.randrange(256) for _ in range(n_ct)), 512)) == 32
        assert len(crypto.mlkem_decaps(bytes(rng.randrange(256) for _ in range(n_dk)), bytes(n_ct), 512)) == 32
    spk, ssk = crypto.slhdsa_keygen("128f", seed=bytes(48))
    ssig = crypto.slhdsa_sign(ssk, b"m", deterministic=True)
    for _ in range(5):
        junk = bytearray(ssig)
        junk[rng.randrange(len(junk))] ^= 1 << rng.randrange(8)
        assert not crypto.slhdsa_verify(spk, b"m", bytes(junk))
