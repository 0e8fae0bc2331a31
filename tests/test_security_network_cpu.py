"""S4: identity management (pins, chains, revocation, OCSP-style cache, connection window) and transport sessions
(PSK and Noise-NN key agreement, AEAD records, replay rejection, rekey, expiry)."""
import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security.network import IdentityManager, TransportError, TransportSecurity, issue_certificate


class Clock:
    def __init__(self, t=1000.0):
        self.t = t

    def __call__(self):
        return self.t


def _chain(clock):
    root_seed, mid_seed, leaf_seed = b"\x01" * 32, b"\x02" * 32, b"\x03" * 32
    root = issue_certificate("Root CA", crypto.ed25519_public_key(root_seed), "Root CA", root_seed, 0, 1e9)
    mid = issue_certificate("Issuing CA", crypto.ed25519_public_key(mid_seed), "Root CA", root_seed, 0, 1e9)
    leaf = issue_certificate("*.models.example", crypto.ed25519_public_key(leaf_seed), "Issuing CA", mid_seed, 500, 5000)
    return root, mid, leaf


def test_chain_verification_pins_revocation_and_hostnames():
    clock = Clock()
    im = IdentityManager(clock=clock)
    root, mid, leaf = _chain(clock)
    assert im.verify_chain([leaf, mid, root]) == (False, "root is not pinned")
    fp = im.pin_certificate(root)
    assert im.verify_pin(fp) and im.verify_chain([leaf, mid, root], "hub.models.example") == (True, "ok")
    assert not im.verify_chain([leaf, mid, root], "models.example")[0]            # wildcard covers one label only
    assert not im.verify_chain([leaf, root])[0]                                    # issuer / subject mismatch
    forged = issue_certificate("*.models.example", leaf.public_key, "Issuing CA", b"\x09" * 32, 500, 5000)
    assert "bad signature" in im.verify_chain([forged, mid, root])[1]
    clock.t = 6000.0
    assert "validity" in im.verify_chain([leaf, mid, root])[1]
    clock.t = 1000.0
    im.add_revocation(mid.fingerprint)
    assert "revoked" in im.verify_chain([leaf, mid, root])[1]
    assert im.revoke_by_subject("Root CA") == 1 and not im.verify_pin(fp)
    assert im.list_pinned()[0]["active"] is False and im.unpin(fp) and not im.unpin(fp)


def test_ocsp_cache_and_connection_window():
    clock = Clock()
    im = IdentityManager(window_s=1.0, limit=3, clock=clock)
    fp = b"\xaa" * 32
    asked = []
    assert im.ocsp_check(fp, lambda f: asked.append(f) or False, ttl=60)
    assert im.ocsp_check(fp, lambda f: asked.append(f) or True, ttl=60)            # served from the cache
    assert len(asked) == 1 and (im.ocsp_hits, im.ocsp_misses) == (1, 1)
    clock.t += 61
    assert not im.ocsp_check(fp, lambda f: True) and im.is_revoked(fp)
    assert [im.connection_allowed() for _ in range(5)] == [True, True, True, False, False]
    clock.t += 1.5
    assert im.connection_allowed() and im.limiter_stats()["blocked"] == 2
    im.enabled = False
    assert all(im.connection_allowed() for _ in range(10))


@pytest.mark.parametrize("cipher", ["chacha20-poly1305", "aes-256-gcm"])
def test_transport_sessions(cipher):
    clock = Clock()
    a, b = TransportSecurity(cipher, clock), TransportSecurity(cipher, clock)
    sa, sb = a.new_session(b"shared secret", True), b.new_session(b"shared secret", False)
    r1 = a.encrypt(sa, b"hello", aad=b"hdr")
    r2 = a.encrypt(sa, b"world")
    assert b.decrypt(sb, r2) == b"world" and b.decrypt(sb, r1, aad=b"hdr") == b"hello"   # out of order is fine
    with pytest.raises(TransportError, match="replayed"):
        b.decrypt(sb, r1, aad=b"hdr")
    tampered = bytearray(a.encrypt(sa, b"x" * 40))
    tampered[20] ^= 1
    with pytest.raises(TransportError, match="authentication"):
        b.decrypt(sb, bytes(tampered))
    with pytest.raises(TransportError, match="authentication"):
        b.decrypt(sb, a.encrypt(sa, b"y"), aad=b"wrong")
    assert a.decrypt(sa, b.encrypt(sb, b"reply")) == b"reply"                            # the other direction
    old = a.encrypt(sa, b"before rekey")
    a.rekey(sa)
    b.rekey(sb)
    assert b.decrypt(sb, a.encrypt(sa, b"after rekey")) == b"after rekey"
    with pytest.raises(TransportError):
        b.decrypt(sb, old)                                                               # old keys are gone
    a.set_timeout(sa, 10)
    clock.t += 11
    with pytest.raises(TransportError, match="timed out"):
        a.encrypt(sa, b"late")
    assert b.cleanup_expired(5) == 1 and b.active_sessions == 0


def test_noise_handshake_agrees_on_keys_and_rejects_a_third_party():
    t1, t2, eve = TransportSecurity(), TransportSecurity(), TransportSecurity()
    m1, st = t1.handshake_initiate(b"\x11" * 32)
    m2, sid2 = t2.handshake_respond(m1, b"\x22" * 32)
    sid1 = t1.handshake_finish(st, m2)
    assert t2.decrypt(sid2, t1.encrypt(sid1, b"ping")) == b"ping"
    assert t1.decrypt(sid1, t2.encrypt(sid2, b"pong")) == b"pong"
    _, sid_e = eve.handshake_respond(m1, b"\x33" * 32)           # same first message, different ephemeral key
    with pytest.raises(TransportError):
        eve.decrypt(sid_e, t1.encrypt(sid1, b"secret"))
    with pytest.raises(TransportError):
        t2.handshake_respond(b"short", b"\x22" * 32)
    assert t1.session_info(sid1)["sent"] == 2
