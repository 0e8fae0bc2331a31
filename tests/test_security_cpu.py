"""Crypto primitives against published test vectors / hashlib, and the host-side security services."""
import hashlib
import hmac as pyhmac

import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security import services as sec


def test_hashes_and_kdfs_match_hashlib():
    for msg in (b"", b"abc", b"a" * 1000, bytes(range(256)) * 3):
        assert crypto.sha256(msg) == hashlib.sha256(msg).digest()
        assert crypto.hmac_sha256(b"key" * 30, msg) == pyhmac.new(b"key" * 30, msg, hashlib.sha256).digest()
    assert crypto.pbkdf2_sha256(b"password", b"salt", 100, 40) == hashlib.pbkdf2_hmac("sha256", b"password", b"salt", 100, 40)
    # RFC 5869 test case 1
    okm = crypto.hkdf_sha256(bytes.fromhex("0b" * 22), bytes.fromhex("000102030405060708090a0b0c"),
                             bytes.fromhex("f0f1f2f3f4f5f6f7f8f9"), 42)
    assert okm.hex() == ("3cb25f25faacd57a90434f64d0362f2a2d2d0a90cf1a5a4c5db02d56ecc4c5bf34007208d5b887185865")


def test_chacha20_poly1305_rfc8439():
    key = bytes(range(0x80, 0xa0))
    nonce = bytes.fromhex("070000004041424344454647")
    aad = bytes.fromhex("50515253c0c1c2c3c4c5c6c7")
    pt = (b"Ladies and Gentlemen of the class of '99: If I could offer you only one tip for the future, "
          b"sunscreen would be it.")
    sealed = crypto.aead_encrypt(key, nonce, pt, aad)
    assert sealed[:16].hex() == "d31a8d34648e60db7b86afbc53ef7ec2"
    assert sealed[-16:].hex() == "1ae10b594f09e26a7e902ecbd0600691"
    assert crypto.aead_decrypt(key, nonce, sealed, aad) == pt
    with pytest.raises(ValueError):
        crypto.aead_decrypt(key, nonce, sealed[:-1] + bytes([sealed[-1] ^ 1]), aad)


def test_x25519_siphash_drbg_guarded():
    # RFC 7748 section 6.1
    a = bytes.fromhex("77076d0a7318a57d3c16c17251b26645df4c2f87ebc0992ab177fba51db92c2a")
    b = bytes.fromhex("5dab087e624a8a4b79e17f8b83800ee66f3bb1292618b6fd1c2f8b27ff88e0eb")
    assert crypto.x25519(a).hex() == "8520f0098930a754748b7ddcb43ef75a0dbf3a0d26381af4eba4a98eaa9b4e6a"
    assert crypto.x25519(a, crypto.x25519(b)) == crypto.x25519(b, crypto.x25519(a))
    assert crypto.x25519(a, crypto.x25519(b)).hex() == "4a5d9d5ba4ce2de1728e3bf480350f25e07e21c947d19e3376f09b3c1e161742"
    # SipHash-2-4 reference vector (key 00..0f, message 00..0e)
    assert crypto.siphash24(bytes(range(16)), bytes(range(15))) == 0xa129ca6149be45e5
    d1, d2 = crypto.HmacDrbg(b"seed"), crypto.HmacDrbg(b"seed")
    assert d1.generate(48) == d2.generate(48) and d1.generate(16) != crypto.HmacDrbg(b"other").generate(16)
    assert crypto.ct_equal(b"abc", b"abc") and not crypto.ct_equal(b"abc", b"abd")
    g = crypto.GuardedBuffer(32)
    g.write(b"secret")
    assert g.check() == 0 and g.read()[:6] == b"secret"
    g.write(b"X" * 4, offset=32)            # overrun into the rear canary
    assert g.check() == 2
    assert g.free() == 2


def test_services(tmp_path):
    f = tmp_path / "model.bin"
    f.write_bytes(b"weights")
    mon = sec.IntegrityMonitor()
    mon.snapshot([str(f)])
    assert mon.verify() == []
    f.write_bytes(b"tampered")
    assert mon.verify() == [str(f)]
    t = [0.0]
    dd = sec.DDoSMitigator(rate=1.0, burst=2.0, ban_after=2, ban_seconds=10.0, clock=lambda: t[0])
    assert [dd.check("c") for _ in range(4)] == [True, True, False, False]
    t[0] = 5.0
    assert not dd.check("c")               # banned
    t[0] = 20.0
    assert dd.check("c") and dd.check("other")
    fw = sec.Firewall()
    fw.add_rule("deny", "10.0.0.0/8")
    fw.add_rule("allow", "0.0.0.0/0", 8080)
    assert fw.decide("10.1.2.3", 8080) == "deny" and fw.decide("1.2.3.4", 8080) == "allow" and fw.decide("1.2.3.4", 22) == "deny"
    v = sec.KeyVault(str(tmp_path / "vault.json"), "passphrase", iterations=1000)
    v.put("hf_token", b"abc123")
    assert sec.KeyVault(str(tmp_path / "vault.json"), "passphrase").get("hf_token") == b"abc123"
    with pytest.raises(ValueError):
        sec.KeyVault(str(tmp_path / "vault.json"), "wrong").get("hf_token")
    log = sec.AuditLogger(str(tmp_path / "audit.jsonl"))
    log.log("admin", "deploy", model="m", version="v2")
    log.log("admin", "rollback", model="m")
    assert log.verify()
    lines = (tmp_path / "audit.jsonl").read_text().splitlines()
    (tmp_path / "audit.jsonl").write_text(lines[0].replace("deploy", "delete") + "\n" + lines[1] + "\n")
    assert not sec.AuditLogger(str(tmp_path / "audit.jsonl")).verify()
    man = sec.sign_update(str(f), b"k" * 32, "1.2.0")
    assert sec.verify_update(str(f), man, b"k" * 32, "1.1.0") and not sec.verify_update(str(f), man, b"x" * 32)
    assert not sec.verify_update(str(f), man, b"k" * 32, "2.0.0")      # downgrade protection
    assert sec.sbom({"torch": "2.11", "left-pad": "0.1"}, {"left-pad==0.1": ["CVE-0"]})["vulnerable"] == ["left-pad"]
    trace = [{"req": True}, {"busy": True}, {"resp": True}]
    assert sec.ltl_check(("always", ("or", ("not", ("ap", "req")), ("eventually", ("ap", "resp")))), trace)
    assert not sec.ltl_check(("always", ("not", ("ap", "busy"))), trace)
    assert sec.ltl_check(("until", ("not", ("ap", "resp")), ("ap", "busy")), trace)

    def parser(b):
        if len(b) > 3 and b[0] == 0xFF:
            raise ValueError("bad header")
    assert any(c["error"] == "ValueError" for c in sec.fuzz(parser, [b"\x00abc", b"hello"], 300))
    assert "API keys are not required" in sec.self_audit({"bind": "0.0.0.0"})
    ks = sec.ApiKeyStore()
    k = ks.create("alice")
    assert ks.check(k) and not ks.check(k, "admin")
    ks.revoke(k)
    assert not ks.check(k)
