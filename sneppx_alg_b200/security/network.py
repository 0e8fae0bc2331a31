"""S4 network security: identity management and transport sessions.

``IdentityManager``: certificate pinning by SHA-256 fingerprint with subject / expiry records, a revocation list, an
OCSP-style result cache with hit / miss counters, chain verification (every certificate is signed by the next one's
Ed25519 key, the last one is a pinned root; expiry and revocation are checked on every link), host-name binding, and
a sliding-window connection limiter. ``TransportSecurity``: numbered sessions keyed from a pre-shared key or from a
Noise-NN-style X25519 handshake (both sides mix the transcript into the keys with HKDF), AEAD records
(ChaCha20-Poly1305 or AES-256-GCM) with per-direction counters as nonces, replay rejection, additional data, rekeying,
idle expiry. All primitives are this package's own (``csrc/host/crypto*.cpp``).
Reference modules of the same purpose: security/network/identity_management.c (pin / verify / revoke / OCSP cache /
DDoS window) and security/network/transport_security.c (sessions, encrypt / decrypt, Noise handshake, rekey, expiry).
"""
from __future__ import annotations

import struct
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from . import crypto


# ----------------------------------------------------------------------------------------------- certificates
@dataclass
class Certificate:
    """A minimal signed identity statement: subject, Ed25519 public key, validity window, issuer's signature over the
    canonical encoding of those fields."""
    subject: str
    public_key: bytes
    not_before: float
    not_after: float
    issuer: str
    signature: bytes = b""

    def tbs(self) -> bytes:
        s, i = self.subject.encode(), self.issuer.encode()
        return struct.pack("<H", len(s)) + s + self.public_key + struct.pack("<ddH", self.not_before, self.not_after, len(i)) + i

    def encode(self) -> bytes:
        return self.tbs() + self.signature

    @property
    def fingerprint(self) -> bytes:
        return crypto.sha256(self.encode())


def issue_certificate(subject: str, public_key: bytes, issuer: str, issuer_seed: bytes, not_before: float,
                      not_after: float) -> Certificate:
    c = Certificate(subject, public_key, not_before, not_after, issuer)
    c.signature = crypto.ed25519_sign(issuer_seed, c.tbs())
    return c


class IdentityManager:
    MAX_CHAIN = 8

    def __init__(self, window_s: float = 1.0, limit: int = 1000, clock: Callable[[], float] = time.time):
        self.clock = clock
        self.pinned: Dict[bytes, dict] = {}
        self.devices: Dict[str, dict] = {}
        self.revoked: set = set()
        self.ocsp_cache: Dict[bytes, Tuple[bool, float]] = {}
        self.ocsp_hits = self.ocsp_misses = 0
        self.window_s, self.limit, self.enabled = window_s, limit, True
        self._events: deque = deque()
        self.blocked = 0

    # ---- pinning
    def pin(self, fingerprint: bytes, subject: str = "", expiry: float = float("inf")) -> None:
        if len(fingerprint) != 32:
            raise ValueError("fingerprint must be a SHA-256 digest")
        self.pinned[bytes(fingerprint)] = {"subject": subject, "expiry": expiry, "active": True}

    def pin_certificate(self, cert: Certificate) -> bytes:
        self.pin(cert.fingerprint, cert.subject, cert.not_after)
        return cert.fingerprint

    def unpin(self, fingerprint: bytes) -> bool:
        return self.pinned.pop(bytes(fingerprint), None) is not None

    def verify_pin(self, fingerprint: bytes) -> bool:
        rec = self.pinned.get(bytes(fingerprint))
        return bool(rec) and rec["active"] and rec["expiry"] > self.clock() and bytes(fingerprint) not in self.revoked

    def revoke_by_subject(self, subject: str) -> int:
        n = 0
        for fp, rec in self.pinned.items():
            if rec["subject"] == subject and rec["active"]:
                rec["active"] = False
                self.revoked.add(fp)
                n += 1
        return n

    def list_pinned(self) -> List[dict]:
        return [{"fingerprint": fp.hex(), **rec} for fp, rec in self.pinned.items()]

    def clear(self) -> None:
        self.pinned.clear()

    # ---- device registry: identities by Ed25519 key (reference: interface_bindings/s4_network.py:53)
    def register(self, device_id: str, public_key: bytes, metadata: Optional[dict] = None) -> None:
        if len(public_key) != 32:
            raise ValueError("an Ed25519 public key has 32 bytes")
        fp = crypto.sha256(bytes(public_key))
        self.devices[device_id] = {"public_key": bytes(public_key), "metadata": dict(metadata or {}),
                                   "fingerprint": fp.hex(), "registered": self.clock()}
        self.pin(fp, subject=device_id)

    def lookup(self, device_id: str) -> Optional[dict]:
        rec = self.devices.get(device_id)
        return dict(rec) if rec and not self.is_revoked(bytes.fromhex(rec["fingerprint"])) else None

    def revoke(self, device_id: str) -> bool:
        rec = self.devices.get(device_id)
        if rec is None or self.is_revoked(bytes.fromhex(rec["fingerprint"])):
            return False
        self.add_revocation(bytes.fromhex(rec["fingerprint"]))
        return True

    def verify_identity(self, device_id: str, challenge: bytes, signature: bytes) -> bool:
        """True when ``signature`` is the registered, unrevoked device's Ed25519 signature over ``challenge``."""
        rec = self.lookup(device_id)
        if rec is None or len(signature) != 64:
            return False
        return crypto.ed25519_verify(rec["public_key"], challenge, signature)

    # ---- revocation / OCSP-style cache
    def add_revocation(self, fingerprint: bytes) -> None:
        self.revoked.add(bytes(fingerprint))

    def is_revoked(self, fingerprint: bytes) -> bool:
        return bytes(fingerprint) in self.revoked

    def ocsp_check(self, fingerprint: bytes, responder: Optional[Callable[[bytes], bool]] = None, ttl: float = 300.0) -> bool:
        """True when the certificate is good. Answers are cached for ``ttl`` seconds; without a cached answer the
        responder (fingerprint -> revoked?) is asked, else the local revocation list decides."""
        fp, now = bytes(fingerprint), self.clock()
        hit = self.ocsp_cache.get(fp)
        if hit and hit[1] > now:
            self.ocsp_hits += 1
            return not hit[0]
        self.ocsp_misses += 1
        revoked = responder(fp) if responder else fp in self.revoked
        self.ocsp_cache[fp] = (bool(revoked), now + ttl)
        if revoked:
            self.revoked.add(fp)
        return not revoked

    # ---- chains
    def verify_chain(self, chain: List[Certificate], hostname: Optional[str] = None) -> Tuple[bool, str]:
        """``chain[0]`` is the leaf, every certificate is signed by the next one, the last must be a pinned root."""
        if not chain or len(chain) > self.MAX_CHAIN:
            return False, "empty chain or chain too long"
        now = self.clock()
        for i, c in enumerate(chain):
            if not (c.not_before <= now < c.not_after):
                return False, f"certificate {i} ({c.subject}) outside its validity window"
            if c.fingerprint in self.revoked:
                return False, f"certificate {i} ({c.subject}) is revoked"
            signer = chain[i + 1] if i + 1 < len(chain) else c
            if c.issuer != signer.subject:
                return False, f"certificate {i} names issuer {c.issuer!r}, next subject is {signer.subject!r}"
            if not crypto.ed25519_verify(signer.public_key, c.tbs(), c.signature):
                return False, f"bad signature on certificate {i} ({c.subject})"
        if not self.verify_pin(chain[-1].fingerprint):
            return False, "root is not pinned"
        if hostname is not None and not self._host_matches(chain[0].subject, hostname):
            return False, f"leaf subject {chain[0].subject!r} does not cover {hostname!r}"
        return True, "ok"

    @staticmethod
    def _host_matches(subject: str, host: str) -> bool:
        subject, host = subject.lower(), host.lower()
        if subject.startswith("*."):
            return host.count(".") == subject.count(".") and host.endswith(subject[1:])
        return subject == host

    # ---- connection limiter
    def connection_allowed(self) -> bool:
        if not self.enabled:
            return True
        now = self.clock()
        while self._events and self._events[0] <= now - self.window_s:
            self._events.popleft()
        if len(self._events) >= self.limit:
            self.blocked += 1
            return False
        self._events.append(now)
        return True

    def limiter_stats(self) -> dict:
        return {"current": len(self._events), "limit": self.limit, "window_s": self.window_s, "blocked": self.blocked}


# ----------------------------------------------------------------------------------------------- transport
@dataclass
class _Session:
    send_key: bytes
    recv_key: bytes
    created: float
    last_used: float
    send_seq: int = 0
    recv_high: int = -1
    recv_seen: set = field(default_factory=set)
    handshake_done: bool = True
    timeout_s: float = float("inf")


class TransportError(RuntimeError):
    pass


class TransportSecurity:
    MAX_SESSIONS, KEY_LEN, NONCE_LEN, REPLAY_WINDOW = 1024, 32, 12, 1024

    def __init__(self, cipher: str = "chacha20-poly1305", clock: Callable[[], float] = time.time):
        assert cipher in ("chacha20-poly1305", "aes-256-gcm")
        self.cipher, self.clock = cipher, clock
        self.sessions: Dict[int, _Session] = {}
        self._next, self.total = 1, 0

    # ---- session setup
    def _add(self, send_key: bytes, recv_key: bytes, done=True) -> int:
        if len(self.sessions) >= self.MAX_SESSIONS:
            raise TransportError("session table is full")
        sid, now = self._next, self.clock()
        self._next += 1
        self.total += 1
        self.sessions[sid] = _Session(send_key, recv_key, now, now, handshake_done=done)
        return sid

    def new_session(self, psk: bytes, initiator: bool = True, context: bytes = b"") -> int:
        """Both ends derive two directional keys from the pre-shared key; ``initiator`` picks which one sends with."""
        a = crypto.hkdf_sha256(psk, b"sneppx-transport", b"i2r" + context, 32)
        b = crypto.hkdf_sha256(psk, b"sneppx-transport", b"r2i" + context, 32)
        return self._add(a, b) if initiator else self._add(b, a)

    # Noise NN (-> e ; <- e, ee): anonymous ephemeral Diffie-Hellman; the transcript hash is mixed into the keys.
    def handshake_initiate(self, seed32: bytes) -> Tuple[bytes, dict]:
        e_pub = crypto.x25519(seed32)
        return e_pub, {"e": seed32, "h": crypto.sha256(b"Noise_NN_25519_sneppx" + e_pub)}

    def handshake_respond(self, msg1: bytes, seed32: bytes) -> Tuple[bytes, int]:
        if len(msg1) != 32:
            raise TransportError("malformed handshake message")
        e_pub = crypto.x25519(seed32)
        h = crypto.sha256(crypto.sha256(b"Noise_NN_25519_sneppx" + msg1) + e_pub)
        dh = crypto.x25519(seed32, msg1)
        k1, k2 = self._split(dh, h)
        return e_pub, self._add(k2, k1)

    def handshake_finish(self, state: dict, msg2: bytes) -> int:
        if len(msg2) != 32:
            raise TransportError("malformed handshake message")
        h = crypto.sha256(state["h"] + msg2)
        dh = crypto.x25519(state["e"], msg2)
        k1, k2 = self._split(dh, h)
        return self._add(k1, k2)

    @staticmethod
    def _split(dh: bytes, h: bytes) -> Tuple[bytes, bytes]:
        if dh == b"\x00" * 32:
            raise TransportError("low-order point in handshake")
        okm = crypto.hkdf_sha256(dh, h, b"sneppx-noise-split", 64)
        return okm[:32], okm[32:]

    # ---- records
    def _aead(self, enc: bool, key: bytes, nonce: bytes, data: bytes, aad: bytes) -> bytes:
        if self.cipher == "aes-256-gcm":
            return crypto.aes256_gcm_encrypt(key, nonce, data, aad) if enc else crypto.aes256_gcm_decrypt(key, nonce, data, aad)
        return crypto.aead_encrypt(key, nonce, data, aad) if enc else crypto.aead_decrypt(key, nonce, data, aad)

    def _get(self, sid: int) -> _Session:
        s = self.sessions.get(sid)
        if s is None:
            raise TransportError(f"unknown session {sid}")
        now = self.clock()
        if now - s.last_used > s.timeout_s:
            del self.sessions[sid]
            raise TransportError(f"session {sid} timed out")
        s.last_used = now
        return s

    def encrypt(self, sid: int, plaintext: bytes, aad: bytes = b"") -> bytes:
        """Record = 8-byte sequence number || ciphertext || tag; the sequence number is the nonce and is authenticated."""
        s = self._get(sid)
        seq = s.send_seq
        s.send_seq += 1
        hdr = struct.pack("<Q", seq)
        return hdr + self._aead(True, s.send_key, b"\x00" * 4 + hdr, plaintext, hdr + aad)

    def decrypt(self, sid: int, record: bytes, aad: bytes = b"") -> bytes:
        s = self._get(sid)
        if len(record) < 8 + 16:
            raise TransportError("record too short")
        hdr = record[:8]
        seq = struct.unpack("<Q", hdr)[0]
        if seq in s.recv_seen or seq <= s.recv_high - self.REPLAY_WINDOW:
            raise TransportError("replayed or stale record")
        try:
            pt = self._aead(False, s.recv_key, b"\x00" * 4 + hdr, record[8:], hdr + aad)
        except Exception as e:  # noqa: BLE001  (authentication failure from either AEAD)
            raise TransportError("record failed authentication") from e
        s.recv_seen.add(seq)
        s.recv_high = max(s.recv_high, seq)
        if len(s.recv_seen) > 2 * self.REPLAY_WINDOW:
            s.recv_seen = {x for x in s.recv_seen if x > s.recv_high - self.REPLAY_WINDOW}
        return pt

    # ---- maintenance
    def rekey(self, sid: int) -> None:
        """Both ends call this at the same point of the stream: keys are ratcheted forward with HKDF and the counters
        restart, so old keys cannot decrypt what follows."""
        s = self._get(sid)
        s.send_key = crypto.hkdf_sha256(s.send_key, b"", b"sneppx-rekey", 32)
        s.recv_key = crypto.hkdf_sha256(s.recv_key, b"", b"sneppx-rekey", 32)
        s.send_seq, s.recv_high, s.recv_seen = 0, -1, set()

    def set_timeout(self, sid: int, seconds: float) -> None:
        self._get(sid).timeout_s = seconds

    def close_session(self, sid: int) -> bool:
        return self.sessions.pop(sid, None) is not None

    def cleanup_expired(self, max_age_s: float) -> int:
        now = self.clock()
        old = [sid for sid, s in self.sessions.items() if now - s.created > max_age_s or now - s.last_used > s.timeout_s]
        for sid in old:
            del self.sessions[sid]
        return len(old)

    def session_info(self, sid: int) -> dict:
        s = self.sessions[sid]
        return {"created": s.created, "last_used": s.last_used, "sent": s.send_seq, "received_high": s.recv_high,
                "handshake_done": s.handshake_done, "cipher": self.cipher}

    @property
    def active_sessions(self) -> int:
        return len(self.sessions)
