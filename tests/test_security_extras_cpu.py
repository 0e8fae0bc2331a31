"""Chaos experiments on host callables, zero-trust decisions, the audit ledger, threat intelligence, incidents,
compliance checks, measured boot and provenance."""
import os

import pytest

from sneppx_alg_b200.security import crypto, extras


def test_chaos_experiment_injects_on_the_host_and_rolls_back():
    calls = {"n": 0, "slept": 0.0}
    store = {}

    def put(k, v):
        calls["n"] += 1
        store[k] = v
        return True
    exp = extras.ChaosExperiment("kv-under-faults", "every acknowledged write is readable", seed=3)
    exp.sleep = lambda s: calls.__setitem__("slept", calls["slept"] + s)
    exp.add_fault("put", extras.Fault("drop", probability=0.3, dropped=False))
    exp.add_fault("put", extras.Fault("delay", probability=0.5, delay_s=0.01))
    flaky_put = exp.wrap("put", put)
    acked = []
    exp.add_probe("acked writes present", lambda: all(store.get(k) == k * 2 for k in acked))

    def workload():
        for k in range(200):
            if flaky_put(k, k * 2):
                acked.append(k)
    assert flaky_put(-1, -2) and calls["n"] == 1                       # not running: no fault
    acked.append(-1)
    rep = exp.run(workload)
    assert rep["hypothesis_valid"] and rep["steady_before"] and rep["steady_after"] and not exp.running
    assert 20 < rep["injected"]["put"] < 200 and 100 < len(acked) < 201 and calls["slept"] > 0
    n = calls["n"]
    assert flaky_put(1000, 2000) and calls["n"] == n + 1               # rolled back: calls go straight through again

    boom = extras.ChaosExperiment("raise", seed=1)
    boom.add_fault("rpc", extras.Fault("exception", error=TimeoutError("injected")))
    rpc = boom.wrap("rpc", lambda: "ok")
    rep = boom.run(lambda: rpc())
    assert not rep["hypothesis_valid"] and "TimeoutError" in rep["workload_error"] and rpc() == "ok"
    with pytest.raises(ValueError):
        boom.add_fault("rpc", extras.Fault("gpu-hang"))


def test_zero_trust_decisions_and_tokens():
    zt = extras.ZeroTrustEngine(b"k" * 32, token_ttl_s=60)
    zt.add_policy(extras.ZTPolicy("/models/prod", ("deploy",), roles=("ml-admin",), min_trust=0.8))
    zt.add_policy(extras.ZTPolicy("/models", ("read", "generate"), roles=("user",), min_trust=0.4))
    good_device, ctx = {"disk_encrypted": True, "managed": True, "patched": True}, {"mfa": True, "known_location": True}
    admin, user = {"id": "ann", "roles": ["user", "ml-admin"]}, {"id": "bob", "roles": ["user"]}
    d = zt.decide(admin, "/models/prod/llama", "deploy", good_device, ctx, now=1000.0)
    assert d["decision"] == "allow" and zt.check_token(d["token"], "/models/prod/llama", "deploy", now=1030.0)
    assert not zt.check_token(d["token"], "/models/prod/llama", "deploy", now=1061.0)            # expired
    assert not zt.check_token(d["token"], "/models/prod/other", "deploy", now=1030.0)            # bound to the resource
    assert not zt.check_token(d["token"][:-2] + "00", "/models/prod/llama", "deploy", now=1030.0)
    assert zt.decide(user, "/models/prod/llama", "deploy", good_device, ctx)["decision"] == "deny"      # role missing
    assert zt.decide(admin, "/models/prod/llama", "deploy", {}, {"mfa": True})["decision"] == "deny"    # posture too weak
    assert zt.decide(user, "/models/x", "generate", {"disk_encrypted": True}, {"mfa": True})["decision"] == "allow"
    assert zt.decide(user, "/models/x", "generate", good_device, {"mfa": True, "recent_failures": 9})["decision"] == "deny"
    assert zt.decide(user, "/secrets", "read", good_device, ctx)["reason"] == "no matching policy" and len(zt.log) == 6


def test_audit_ledger_quorum_and_tamper_detection():
    seeds = {n: os.urandom(32) for n in ("a", "b", "c", "d")}
    ledger = extras.AuditLedger({n: crypto.ed25519_public_key(s) for n, s in seeds.items()})
    assert ledger.quorum == 3
    for blk in range(3):
        for i in range(blk + 2):
            ledger.append({"event": "deploy", "model": f"m{blk}", "i": i})
        b = ledger.propose(now=100.0 + blk)
        for n in ("a", "b"):
            ledger.vote(b, n, seeds[n])
        assert not ledger.commit(b)                                       # two votes of four: below quorum
        b["votes"]["mallory"] = b["votes"]["a"]                           # unknown validator does not count
        assert not ledger.commit(b)
        ledger.vote(b, "c", seeds["c"])
        assert ledger.commit(b) and not ledger.pending
    assert ledger.verify() and len(ledger.blocks) == 3
    ledger.blocks[1]["records"][0]["model"] = "evil"
    assert not ledger.verify()
    ledger.blocks[1]["records"][0]["model"] = "m1"
    assert ledger.verify()
    ledger.blocks[1], ledger.blocks[2] = ledger.blocks[2], ledger.blocks[1]
    assert not ledger.verify()
    assert extras.merkle_root([b"a", b"b", b"c"]) != extras.merkle_root([b"a", b"b"]) != extras.merkle_root([b"b", b"a"])


def test_threat_intel_incidents_compliance():
    ti = extras.ThreatIntel()
    ti.add("ip", "203.0.113.9", 0.6, "feed-a", ttl_s=100, now=0)
    ti.add("ip", "203.0.113.9", 0.4, "feed-b", ttl_s=100, now=10)
    ti.add("sha256", "AB" * 32, 0.9, "sandbox", now=0)
    m = ti.match({"ip": "203.0.113.9", "sha256": "ab" * 32}, now=50)
    assert len(m["hits"]) == 2 and abs(m["score"] - (1 - 0.4 * 0.1)) < 1e-9 and m["hits"][0]["sources"] == ["feed-a", "feed-b"]
    assert ti.match({"ip": "198.51.100.1"}, now=50)["score"] == 0.0
    assert ti.expire(now=200) == 1 and ti.match({"ip": "203.0.113.9"}, now=200)["hits"] == []

    im = extras.IncidentManager()
    blocked = []
    im.register_playbook("credential-leak", [("revoke", lambda inc: "revoked"), ("block", lambda inc: blocked.append(inc["id"]) or "blocked"),
                                             ("notify", lambda inc: 1 / 0), ("never", lambda inc: "unreachable")])
    i = im.open("credential-leak", "high", "API key in a public log", now=1.0)
    im.add_evidence(i, "log.txt", b"key=abc")
    res = im.run_playbook(i)
    assert [r["ok"] for r in res] == [True, True, False] and blocked == [i] and "ZeroDivisionError" in res[2]["error"]
    im.advance(i, "triaged"); im.advance(i, "contained", "key revoked")
    with pytest.raises(ValueError):
        im.advance(i, "open")
    im.advance(i, "resolved")
    assert im.incidents[i]["state"] == "resolved" and im.incidents[i]["evidence"][0]["sha256"] == crypto.sha256(b"key=abc").hex()
    with pytest.raises(ValueError):
        im.open("x", "urgent", "bad severity")

    cfg = {"encrypt_checkpoints": True, "tls": True, "api_keys_required": True, "audit_log": "a.log", "retention_days": 30}
    r = extras.compliance_report(cfg, "gdpr")
    assert not r["compliant"] and r["missing"] == ["erasure"] and r["passed"] == 5
    cfg.update(supports_erasure=True, incident_contact="sec@example.org")
    assert extras.compliance_report(cfg, "gdpr")["compliant"] and extras.compliance_report(cfg, "hipaa")["compliant"]
    assert set(extras.compliance_report(cfg, "pci_dss")["missing"]) == {"key_rotation", "mfa", "vulnerability_management"}
    with pytest.raises(ValueError):
        extras.compliance_report(cfg, "iso9001")


def test_measured_boot_and_provenance():
    seed = os.urandom(32)
    pub = crypto.ed25519_public_key(seed)
    comps = [b"bootloader v3", b"kernel 6.1", b"libsneppx_b200.so"]
    mb = extras.MeasuredBoot()
    for n, c in zip(("boot", "kernel", "runtime"), comps):
        mb.extend(n, c)
    nonce = os.urandom(16)
    q = mb.quote(seed, nonce)
    assert extras.MeasuredBoot.verify_quote(q, pub, nonce, comps)
    assert not extras.MeasuredBoot.verify_quote(q, pub, os.urandom(16), comps)                   # replay with another nonce
    assert not extras.MeasuredBoot.verify_quote(q, pub, nonce, [comps[1], comps[0], comps[2]])   # order matters
    assert not extras.MeasuredBoot.verify_quote(q, pub, nonce, comps[:2] + [b"patched runtime"])

    arts = {"libsneppx_b200.so": b"\x7fELF...", "weights.sneppx": os.urandom(64)}
    att = extras.provenance_attestation(arts, "ci-runner-7", "git:abc123", seed)
    assert extras.verify_provenance(att, arts, pub)
    assert not extras.verify_provenance(att, {**arts, "weights.sneppx": b"swapped"}, pub)
    assert not extras.verify_provenance(att, {"libsneppx_b200.so": arts["libsneppx_b200.so"]}, pub)
    assert not extras.verify_provenance({**att, "builder": "someone-else"}, arts, pub)
