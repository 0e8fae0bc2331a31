"""S6 extensions (``security/vault_ext.py``): secret sharing, the key store, ceremonies and rotation, the policy
language, the threat graph, dashboard and compliance reports."""
import json
import os

import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security import vault_ext as vx


def test_shamir_any_k_shares_rebuild_fewer_do_not():
    secret = os.urandom(48)
    shares = vx.shamir_split(secret, 9, 5)
    assert len(shares) == 9 and all(len(s) == 49 for s in shares) and [s[0] for s in shares] == list(range(1, 10))
    import itertools
    for combo in list(itertools.combinations(shares, 5))[::17]:
        assert vx.shamir_reconstruct(combo) == secret
    assert vx.shamir_reconstruct(shares) == secret and vx.shamir_reconstruct(shares[:4]) != secret
    assert vx.shamir_reconstruct(vx.shamir_split(b"x", 1, 1)) == b"x"
    # k = 2 with a fixed polynomial: share(x) = s + a x in GF(256)
    sh = vx.shamir_split(b"\x05", 3, 2, rng=lambda n: b"\x03" * n)
    assert [s[1] for s in sh] == [5 ^ 3, 5 ^ 6, 5 ^ 5]
    with pytest.raises(ValueError):
        vx.shamir_split(b"s", 3, 4)
    with pytest.raises(ValueError):
        vx.shamir_reconstruct([shares[0], shares[0]])
    # field sanity: every non-zero element has an inverse
    assert all(vx._gf_mul(a, vx._gf_div(1, a)) == 1 for a in range(1, 256))


def test_key_store_use_by_id_wrap_and_export_rules():
    ks = vx.KeyStore(capacity=4)
    kid = ks.generate_key("aes256")
    with pytest.raises(vx.KeyStoreError, match="not exportable"):
        ks.load_key(kid)
    sealed = ks.encrypt(kid, b"payload", b"aad")
    assert ks.decrypt(kid, sealed, b"aad") == b"payload" and ks.key_info(kid)["uses"] == 2
    with pytest.raises(ValueError):
        ks.decrypt(kid, sealed, b"other aad")
    ks.store_key(b"mac", b"k" * 32, "hmac")
    assert ks.mac(b"mac", b"m") == crypto.hmac_sha256(b"k" * 32, b"m") and ks.load_key(b"mac") == b"k" * 32
    sk = ks.generate_key("ed25519-seed", b"signer")
    assert crypto.ed25519_verify(ks.public_key(sk), b"msg", ks.sign(sk, b"msg"))
    with pytest.raises(vx.KeyStoreError):
        ks.sign(kid, b"msg")
    wrap = ks.generate_key("chacha20", b"kek", exportable=True)
    blob = ks.wrap_key(kid, wrap)
    other = vx.KeyStore()
    other.store_key(b"kek", ks.load_key(b"kek"), "chacha20")
    other.unwrap_key(blob, b"kek", kid)
    assert other.decrypt(kid, sealed, b"aad") == b"payload" and other.key_info(kid) == {**other.key_info(kid), "kind": "aes256", "exportable": False}
    with pytest.raises(vx.KeyStoreError, match="authenticate"):
        other.unwrap_key(blob[:-1] + bytes([blob[-1] ^ 1]), b"kek", b"new")
    with pytest.raises(vx.KeyStoreError, match="full"):
        ks.generate_key()
        ks.generate_key()
    assert ks.delete_key(b"mac") and not ks.delete_key(b"mac") and b"mac" not in ks.list_keys()
    with pytest.raises(vx.KeyStoreError):
        ks.generate_key("rsa")
    # a sealed entry is bound to its id: moving it under another id fails to open
    ks._keys[b"moved"] = ks._keys.pop(kid)
    with pytest.raises(ValueError):
        ks.encrypt(b"moved", b"x")


def test_key_ceremony_and_rotation():
    now = [0.0]
    store = vx.KeyStore()
    cer = vx.KeyCeremony(participants=5, required=3, timeout_s=600.0, clock=lambda: now[0])
    tokens = {n: os.urandom(16) for n in ("ann", "bob", "cat", "dan", "eve")}
    for n, t in tokens.items():
        cer.enroll(n, t)
    with pytest.raises(ValueError):
        cer.enroll("zed", b"t")
    assert cer.approve(tokens["ann"]) and not cer.approve(tokens["ann"]) and not cer.approve(b"stranger")
    with pytest.raises(vx.KeyStoreError, match="1 of 3"):
        cer.execute(store)
    assert cer.approve(tokens["bob"]) and cer.approve(tokens["eve"])
    assert cer.status() == {"state": "open", "approved": 3, "present": 5, "required": 3}
    kid, shares = cer.execute(store, "aes256", b"root-key")
    assert sorted(shares) == ["ann", "bob", "eve"] and cer.status()["state"] == "executed" and not cer.cancel()
    with pytest.raises(vx.KeyStoreError, match="not exportable"):
        store.load_key(kid)
    rebuilt = vx.shamir_reconstruct(list(shares.values()))
    probe = store.encrypt(kid, b"p")
    other = vx.KeyStore()
    other.store_key(b"r", rebuilt)
    assert other.decrypt(b"r", probe) == b"p"                                  # the shares rebuild the very key in the store
    late = vx.KeyCeremony(3, clock=lambda: now[0])
    late.enroll("a", b"a")
    now[0] += 4000.0
    assert not late.approve(b"a") and late.status()["state"] == "expired"
    c2 = vx.KeyCeremony(2, clock=lambda: now[0])
    assert c2.required == 2 and c2.cancel() and c2.status()["state"] == "cancelled"
    rotated = []
    rot = vx.KeyRotationScheduler(100.0, rotate=rotated.append, clock=lambda: now[0])
    assert not rot.check() and rot.remaining() == 100.0
    now[0] += 100.0
    assert rot.check() and rotated == [1] and rot.remaining() == 100.0 and not rot.check()
    rot.set_auto(False)
    now[0] += 150.0
    assert rot.check() and rot.check() and rotated == [1] and rot.force_rotate() == 2 and rotated == [1, 2] and rot.count == 2


def test_policy_language_compiles_and_decides():
    p = vx.PolicyDSL(['allow role:admin * *',
                      'allow role:ml-* deploy model/* if env == "staging" or (hour >= 8 and hour < 18)',
                      'deny * delete model/prod-* if not mfa',
                      'allow * delete model/*',
                      'allow * read * if region in "eu,us" and path matches "^/public/"'])
    code = p.compile()
    assert isinstance(code, bytes) and code[-1] == vx.OP_RET_DENY and p.rule_count() == 5 and p.validate() == []
    ev = p.evaluate
    assert ev("role:admin", "anything", "at/all")
    assert ev("role:ml-eng", "deploy", "model/a", env="staging", hour=23) and ev("role:ml-eng", "deploy", "model/a", env="prod", hour=9)
    assert not ev("role:ml-eng", "deploy", "model/a", env="prod", hour=20) and not ev("role:ml-eng", "deploy", "data/a", env="staging")
    assert not ev("u", "delete", "model/prod-7") and not ev("u", "delete", "model/prod-7", mfa=False) and ev("u", "delete", "model/prod-7", mfa=True)
    assert ev("u", "delete", "model/dev-1") and not ev("u", "write", "model/dev-1")
    assert ev("u", "read", "x", region="eu", path="/public/a") and not ev("u", "read", "x", region="cn", path="/public/a")
    assert not ev("u", "read", "x", region="eu", path="/private/a") and not ev("u", "read", "x")            # missing attributes
    assert vx.PolicyDSL.run(code, {"subject": "role:admin", "action": "a", "resource": "r"})
    p.add_rule("allow * write *")
    assert ev("u", "write", "model/dev-1")
    p.set_rule(5, "deny * write *")
    assert not ev("u", "write", "model/dev-1") and p.remove_rule(5) and not p.remove_rule(9)
    shadow = vx.PolicyDSL(["deny * * *", "allow role:admin * *"])
    assert shadow.validate() == ["rule 1 is shadowed by rule 0"] and not shadow.evaluate("role:admin", "a", "b")
    assert not vx.PolicyDSL().evaluate("a", "b", "c")                                                      # default deny
    for bad in ("permit a b c", "allow a b", "allow a b c if", "allow a b c if (x == 1", "allow a b c if x ==", "allow a b c if 1 2"):
        with pytest.raises(vx.PolicyError):
            vx.PolicyDSL([bad])
    assert vx.PolicyDSL(['allow * * * if note == "say \\"hi\\""']).evaluate("s", "a", "r", note='say "hi"')
    assert vx.PolicyDSL(["allow * * * if x < 5"]).evaluate("s", "a", "r", x="text") is False                # type mismatch is false


def test_threat_graph_dashboard_and_reports(tmp_path):
    g = vx.ThreatGraph()
    for a, b, l in (("internet", "gateway", "exposed port"), ("gateway", "api", "stolen token"), ("gateway", "worker", "ssrf"),
                    ("api", "vault", "over-broad role"), ("worker", "api", "lateral move"), ("laptop", "vault", "phished admin")):
        g.add_edge(a, b, l)
    paths = g.attack_paths("internet", "vault")
    assert paths == [["internet", "gateway", "api", "vault"], ["internet", "gateway", "worker", "api", "vault"]]
    assert g.choke_points("internet", "vault") == ["api", "gateway"] and g.attack_paths("vault", "internet") == []
    dot = g.export_dot(str(tmp_path / "t.dot"))
    assert '"api" -> "vault" [label="over-broad role"];' in dot and (tmp_path / "t.dot").read_text() == dot
    assert g.edge_count() == 6 and g.remove_edge("laptop", "vault") and not g.remove_edge("laptop", "vault") and "laptop" not in g.nodes()
    g.clear()
    assert g.edge_count() == 0
    now = [5.0]
    d = vx.SecurityDashboard("SOC", clock=lambda: now[0])
    d.add_widget("blocked", "counter")
    d.add_widget("risk", "gauge", 0.2)
    d.add_widget("alerts", "table")
    assert d.update('{"blocked": 3, "risk": 0.7, "unknown": 1}') == 2 and d.update({"blocked": 2, "alerts": [["<b>x</b>", 1]]}) == 2
    st = json.loads(d.status())
    assert st["widgets"]["blocked"]["data"] == 5 and st["widgets"]["risk"]["data"] == 0.7 and st["updated"] == 5.0
    page = d.render_html()
    assert "&lt;b&gt;x&lt;/b&gt;" in page and "<b>x</b>" not in page and page.startswith("<!doctype html>")
    assert d.remove_widget("risk") and not d.remove_widget("risk")
    with pytest.raises(ValueError):
        d.add_widget("w", "dial")
    rep = vx.ComplianceReportBuilder("Acme (EU)")
    rep.add_finding("CC6.1", "pass", "logical access controls")
    rep.add_finding("CC6.6", "partial", "boundary protection")
    rep.add_finding("CC7.2", "fail", "monitoring of anomalies")
    rep.add_finding("CC9.9", "n/a")
    assert rep.score() == pytest.approx(0.5)
    text = rep.generate("soc2", str(tmp_path / "r.txt"))
    assert "SOC 2 Type II" in text and "[FAIL   ] CC7.2" in text and "Score: 50.0%" in text
    assert json.loads(rep.generate("iso27001", fmt="json"))["findings"][1]["status"] == "partial"
    size = rep.generate_pdf("soc2", str(tmp_path / "r.pdf"))
    raw = (tmp_path / "r.pdf").read_bytes()
    assert size == len(raw) and raw.startswith(b"%PDF-1.4") and raw.rstrip().endswith(b"%%EOF") and b"Acme \\(EU\\)" in raw
    xref = int(raw.rsplit(b"startxref\n", 1)[1].split()[0])
    assert raw[xref:xref + 4] == b"xref"
    first_obj = int(raw[xref:].split(b"\n")[3].split()[0])
    assert raw[first_obj:first_obj + 7] == b"1 0 obj"
    with pytest.raises(ValueError):
        rep.generate("nist")
    with pytest.raises(ValueError):
        rep.add_finding("X", "maybe")
