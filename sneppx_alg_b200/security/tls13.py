"""TLS 1.3 (RFC 8446) client and server as sans-I/O state machines, with a socket wrapper.

Scope, chosen so that every primitive is one this package already owns and every message can be checked against another
implementation (the tests run both roles against the OpenSSL command-line programs):

* cipher suites TLS_CHACHA20_POLY1305_SHA256 and TLS_AES_128_GCM_SHA256; key exchange x25519;
* server authentication by an Ed25519 certificate (signature scheme ed25519), with the client either pinning public
  keys or walking an Ed25519-signed chain to a trusted root; a DER reader / writer for exactly the X.509 fields that
  needs (``make_certificate`` / ``parse_certificate``);
* external pre-shared keys and session resumption, both in psk_dhe_ke mode (binders, NewSessionTicket, ticket age);
* the record layer (fragmentation, coalesced and split handshake messages, inner content type and padding, sequence
  numbers, the ignored ChangeCipherSpec of middlebox-compatibility mode), alerts, close_notify, KeyUpdate in both
  directions.

Not covered: HelloRetryRequest (a peer that offers no x25519 share is refused with handshake_failure), client
certificates, 0-RTT data, SHA-384 suites, RSA / ECDSA certificates.

The key schedule is ``network_ext.Tls13KeySchedule``. The reference's transport layer
(security/network/transport_security.c:95-260: sessions keyed by a PSK, encrypt / decrypt with a rekey counter, session
info) has no handshake or record format of its own to match; this module supplies the standard ones.
"""
from __future__ import annotations

import hashlib
import os
import socket
import struct
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from . import crypto
from .network_ext import (TLS_AES_128_GCM_SHA256, TLS_CHACHA20_POLY1305_SHA256, Tls13KeySchedule, hkdf_expand_label)

# content types, handshake types, extensions, alerts
CT_CCS, CT_ALERT, CT_HANDSHAKE, CT_APPDATA = 20, 21, 22, 23
HS_CLIENT_HELLO, HS_SERVER_HELLO, HS_NEW_SESSION_TICKET, HS_ENCRYPTED_EXTENSIONS = 1, 2, 4, 8
HS_CERTIFICATE, HS_CERTIFICATE_REQUEST, HS_CERTIFICATE_VERIFY, HS_FINISHED, HS_KEY_UPDATE = 11, 13, 15, 20, 24
EXT_SERVER_NAME, EXT_SUPPORTED_GROUPS, EXT_SIGNATURE_ALGORITHMS, EXT_ALPN = 0, 10, 13, 16
EXT_PRE_SHARED_KEY, EXT_EARLY_DATA, EXT_SUPPORTED_VERSIONS, EXT_PSK_MODES, EXT_KEY_SHARE = 41, 42, 43, 45, 51
EXT_QUIC_TRANSPORT_PARAMETERS = 57
GROUP_X25519, SIG_ED25519, PSK_DHE_KE = 0x001D, 0x0807, 1
ALERT_CLOSE_NOTIFY, ALERT_UNEXPECTED_MESSAGE, ALERT_BAD_RECORD_MAC, ALERT_HANDSHAKE_FAILURE = 0, 10, 20, 40
ALERT_BAD_CERTIFICATE, ALERT_ILLEGAL_PARAMETER, ALERT_DECODE_ERROR, ALERT_DECRYPT_ERROR = 42, 47, 50, 51
ALERT_PROTOCOL_VERSION, ALERT_INTERNAL_ERROR, ALERT_MISSING_EXTENSION, ALERT_UNKNOWN_PSK_IDENTITY = 70, 80, 109, 115
ALERT_NO_APPLICATION_PROTOCOL = 120
HRR_RANDOM = bytes.fromhex("cf21ad74e59a6111be1d8c021e65b891c2a211167abb8c5e079e09e2c8a8339c")
MAX_FRAGMENT = 16384
SUITES = (TLS_CHACHA20_POLY1305_SHA256, TLS_AES_128_GCM_SHA256)


class TlsError(RuntimeError):
    """A fatal condition; ``alert`` is the description code sent to (or received from) the peer."""

    def __init__(self, message: str, alert: int = ALERT_INTERNAL_ERROR, received: bool = False):
        super().__init__(message)
        self.alert, self.received = alert, received


# ------------------------------------------------------------------------------------------------------------ DER / X.509
OID_ED25519 = bytes.fromhex("2b6570")                      # 1.3.101.112
OID_COMMON_NAME = bytes.fromhex("550403")
OID_SUBJECT_ALT_NAME = bytes.fromhex("551d11")
OID_BASIC_CONSTRAINTS = bytes.fromhex("551d13")


def _der(tag: int, body: bytes) -> bytes:
    n = len(body)
    if n < 0x80:
        return bytes([tag, n]) + body
    ln = n.to_bytes((n.bit_length() + 7) // 8, "big")
    return bytes([tag, 0x80 | len(ln)]) + ln + body


def _der_int(v: int) -> bytes:
    return _der(0x02, v.to_bytes(v.bit_length() // 8 + 1, "big"))


def _der_read(buf: bytes, pos: int) -> Tuple[int, bytes, int, int]:
    """(tag, content, start of this element, position after it); definite lengths only."""
    start = pos
    if pos + 2 > len(buf):
        raise ValueError("truncated DER")
    tag, n = buf[pos], buf[pos + 1]
    pos += 2
    if n & 0x80:
        k = n & 0x7F
        if k == 0 or k > 4 or pos + k > len(buf):
            raise ValueError("bad DER length")
        n = int.from_bytes(buf[pos:pos + k], "big")
        pos += k
    if pos + n > len(buf):
        raise ValueError("truncated DER")
    return tag, buf[pos:pos + n], start, pos + n


def _der_children(body: bytes) -> List[Tuple[int, bytes, bytes]]:
    """(tag, content, full encoding) of each element of a constructed value."""
    out, pos = [], 0
    while pos < len(body):
        tag, content, start, pos = _der_read(body, pos)
        out.append((tag, content, body[start:pos]))
    return out


def _name(common_name: str) -> bytes:
    return _der(0x30, _der(0x31, _der(0x30, _der(0x06, OID_COMMON_NAME) + _der(0x0C, common_name.encode()))))


def _time(t: float) -> bytes:
    g = time.gmtime(t)                                        # RFC 5280: UTCTime through 2049, GeneralizedTime after
    if g.tm_year < 2050:
        return _der(0x17, time.strftime("%y%m%d%H%M%SZ", g).encode())
    return _der(0x18, time.strftime("%Y%m%d%H%M%SZ", g).encode())


def _parse_time(tag: int, body: bytes) -> float:
    import calendar
    s = body.decode()
    if tag == 0x17:                                                                       # UTCTime: two-digit year
        s = ("19" if int(s[:2]) >= 50 else "20") + s
    return calendar.timegm(time.strptime(s, "%Y%m%d%H%M%SZ"))


def make_certificate(subject_seed: bytes, subject: str, issuer_seed: Optional[bytes] = None, issuer: Optional[str] = None,
                     days: float = 365.0, dns_names: Sequence[str] = (), ca: bool = False, serial: Optional[int] = None,
                     not_before: Optional[float] = None) -> bytes:
    """A DER X.509 v3 certificate for the Ed25519 key of ``subject_seed``, signed by ``issuer_seed`` (itself when
    omitted: self-signed)."""
    issuer_seed, issuer = issuer_seed or subject_seed, issuer or subject
    alg = _der(0x30, _der(0x06, OID_ED25519))
    start = time.time() - 300 if not_before is None else not_before
    exts = b""
    if dns_names:
        san = _der(0x30, b"".join(_der(0x82, d.encode()) for d in dns_names))
        exts += _der(0x30, _der(0x06, OID_SUBJECT_ALT_NAME) + _der(0x04, san))
    if ca:
        exts += _der(0x30, _der(0x06, OID_BASIC_CONSTRAINTS) + _der(0x01, b"\xff") + _der(0x04, _der(0x30, _der(0x01, b"\xff"))))
    tbs = _der(0x30, _der(0xA0, _der_int(2)) + _der_int(serial if serial is not None else int.from_bytes(os.urandom(8), "big") >> 1)
               + alg + _name(issuer) + _der(0x30, _time(start) + _time(start + days * 86400)) + _name(subject)
               + _der(0x30, alg + _der(0x03, b"\0" + crypto.ed25519_public_key(subject_seed)))
               + (_der(0xA3, _der(0x30, exts)) if exts else b""))
    return _der(0x30, tbs + alg + _der(0x03, b"\0" + crypto.ed25519_sign(issuer_seed, tbs)))


def parse_certificate(der: bytes) -> dict:
    """The fields chain validation needs: the signed bytes, signature and its algorithm, names, validity, the subject's
    key and its algorithm, DNS names, the CA flag."""
    try:
        return _parse_certificate(der)
    except (IndexError, UnicodeDecodeError, TypeError):
        raise ValueError("not a certificate") from None


def _parse_certificate(der: bytes) -> dict:
    tag, cert, _, end = _der_read(der, 0)
    if tag != 0x30 or end != len(der):
        raise ValueError("not a certificate")
    (t_tag, tbs_body, tbs), (_, sig_alg, _), (s_tag, sig, _) = _der_children(cert)[:3]
    if t_tag != 0x30 or s_tag != 0x03:
        raise ValueError("not a certificate")
    f = _der_children(tbs_body)
    if f[0][0] == 0xA0:
        f = f[1:]                                                                        # explicit version
    serial, _inner_alg, issuer, validity, subject, spki = f[:6]

    def common_name(name_body: bytes) -> str:
        for _, rdn, _ in _der_children(name_body):
            for _, atv, _ in _der_children(rdn):
                kv = _der_children(atv)
                if kv[0][1] == OID_COMMON_NAME:
                    return kv[1][1].decode(errors="replace")
        return ""

    (nb_tag, nb, _), (na_tag, na, _) = _der_children(validity[1])
    spki_alg, spki_key = _der_children(spki[1])
    out = {"tbs": tbs, "signature": sig[1:], "signature_oid": _der_children(sig_alg)[0][1], "serial": int.from_bytes(serial[1], "big"),
           "issuer": common_name(issuer[1]), "subject": common_name(subject[1]), "issuer_der": issuer[2], "subject_der": subject[2],
           "not_before": _parse_time(nb_tag, nb), "not_after": _parse_time(na_tag, na),
           "key_oid": _der_children(spki_alg[1])[0][1], "public_key": spki_key[1][1:], "dns_names": [], "ca": False}
    for tag, body, _ in f[6:]:
        if tag != 0xA3:
            continue
        for _, ext, _ in _der_children(_der_children(body)[0][1]):
            parts = _der_children(ext)
            oid, value = parts[0][1], parts[-1][1]
            if oid == OID_SUBJECT_ALT_NAME:
                out["dns_names"] = [c.decode() for t, c, _ in _der_children(_der_children(value)[0][1]) if t == 0x82]
            elif oid == OID_BASIC_CONSTRAINTS:
                inner = _der_children(_der_children(value)[0][1])
                out["ca"] = bool(inner and inner[0][0] == 0x01 and inner[0][1] != b"\0")
    return out


def _host_matches(pattern: str, host: str) -> bool:
    pattern, host = pattern.lower(), host.lower()
    if pattern.startswith("*."):
        return "." in host and host.split(".", 1)[1] == pattern[2:]
    return pattern == host


def verify_chain(chain: Sequence[bytes], trusted_roots: Iterable[bytes], hostname: Optional[str] = None,
                 now: Optional[float] = None) -> bytes:
    """Walk ``chain`` (leaf first) to a certificate in ``trusted_roots`` (DER): each link's Ed25519 signature, validity
    window and CA flag, and the leaf's DNS names (or common name) against ``hostname``. Returns the leaf's public key."""
    now = time.time() if now is None else now
    roots = [parse_certificate(r) for r in trusted_roots]
    try:
        certs = [parse_certificate(c) for c in chain]
    except ValueError as e:
        raise TlsError(f"unreadable certificate in the chain: {e}", ALERT_BAD_CERTIFICATE) from None
    if not certs:
        raise TlsError("empty certificate chain", ALERT_BAD_CERTIFICATE)
    for c in certs:
        if c["key_oid"] != OID_ED25519 or c["signature_oid"] != OID_ED25519:
            raise TlsError("only Ed25519 certificates are supported", ALERT_BAD_CERTIFICATE)
        if not c["not_before"] <= now <= c["not_after"]:
            raise TlsError(f"certificate for {c['subject']!r} is outside its validity window", ALERT_BAD_CERTIFICATE)
    if hostname is not None:
        names = certs[0]["dns_names"] or [certs[0]["subject"]]
        if not any(_host_matches(n, hostname) for n in names):
            raise TlsError(f"certificate names {names} do not cover {hostname!r}", ALERT_BAD_CERTIFICATE)
    for i, c in enumerate(certs):
        for r in roots:
            if r["subject_der"] == c["issuer_der"] and crypto.ed25519_verify(r["public_key"], c["tbs"], c["signature"]):
                if not r["not_before"] <= now <= r["not_after"]:
                    raise TlsError("trusted root is outside its validity window", ALERT_BAD_CERTIFICATE)
                return certs[0]["public_key"]
        if i + 1 == len(certs):
            break
        parent = certs[i + 1]
        if not parent["ca"] or parent["subject_der"] != c["issuer_der"] or \
                not crypto.ed25519_verify(parent["public_key"], c["tbs"], c["signature"]):
            raise TlsError("broken certificate chain", ALERT_BAD_CERTIFICATE)
    raise TlsError("certificate chain does not reach a trusted root", ALERT_BAD_CERTIFICATE)


# ------------------------------------------------------------------------------------------------------------ wire helpers
def _v8(b: bytes) -> bytes:
    return bytes([len(b)]) + b


def _v16(b: bytes) -> bytes:
    return struct.pack(">H", len(b)) + b


def _v24(b: bytes) -> bytes:
    return len(b).to_bytes(3, "big") + b


class _Reader:
    def __init__(self, buf: bytes):
        self.buf, self.pos = buf, 0

    def take(self, n: int) -> bytes:
        if n < 0 or self.pos + n > len(self.buf):
            raise TlsError("message shorter than its length fields say", ALERT_DECODE_ERROR)
        self.pos += n
        return self.buf[self.pos - n:self.pos]

    def u8(self) -> int:
        return self.take(1)[0]

    def u16(self) -> int:
        return struct.unpack(">H", self.take(2))[0]

    def u32(self) -> int:
        return struct.unpack(">I", self.take(4))[0]

    def vec(self, len_bytes: int) -> bytes:
        return self.take(int.from_bytes(self.take(len_bytes), "big"))

    def done(self) -> bool:
        return self.pos == len(self.buf)


def _handshake(msg_type: int, body: bytes) -> bytes:
    return bytes([msg_type]) + _v24(body)


def _extensions(pairs: Sequence[Tuple[int, bytes]]) -> bytes:
    return _v16(b"".join(struct.pack(">H", t) + _v16(d) for t, d in pairs))


def _parse_extensions(r: _Reader) -> Dict[int, bytes]:
    out: Dict[int, bytes] = {}
    if r.done():
        return out
    er = _Reader(r.vec(2))
    while not er.done():
        t = er.u16()
        if t in out:
            raise TlsError("extension sent twice", ALERT_ILLEGAL_PARAMETER)
        out[t] = er.vec(2)
    return out


def _aead_seal(suite: int, key: bytes, nonce: bytes, data: bytes, aad: bytes) -> bytes:
    if suite == TLS_CHACHA20_POLY1305_SHA256:
        return crypto.aead_encrypt(key, nonce, data, aad)
    from ..utils.quic_protection import aes128_gcm_encrypt
    return aes128_gcm_encrypt(key, nonce, data, aad)


def _aead_open(suite: int, key: bytes, nonce: bytes, data: bytes, aad: bytes) -> bytes:
    try:
        if suite == TLS_CHACHA20_POLY1305_SHA256:
            return crypto.aead_decrypt(key, nonce, data, aad)
        from ..utils.quic_protection import aes128_gcm_decrypt
        return aes128_gcm_decrypt(key, nonce, data, aad)
    except Exception as e:
        raise TlsError("record failed authentication", ALERT_BAD_RECORD_MAC) from e


class _RecordLayer:
    """Framing, protection and sequence numbers of one connection (RFC 8446 section 5)."""

    def __init__(self):
        self.suite = None
        self.read_key = self.write_key = None             # (key, iv) once a direction is protected
        self.read_seq = self.write_seq = 0
        self.inbuf = bytearray()
        self.pad_to = 0                                   # pad application records up to a multiple of this many bytes

    def set_read(self, suite: int, key_iv: Tuple[bytes, bytes]) -> None:
        self.suite, self.read_key, self.read_seq = suite, key_iv, 0

    def set_write(self, suite: int, key_iv: Tuple[bytes, bytes]) -> None:
        self.suite, self.write_key, self.write_seq = suite, key_iv, 0

    def seal(self, content_type: int, data: bytes) -> bytes:
        out = bytearray()
        for off in range(0, max(len(data), 1), MAX_FRAGMENT):
            frag = data[off:off + MAX_FRAGMENT]
            if self.write_key is None:
                out += struct.pack(">BHH", content_type, 0x0303, len(frag)) + frag
                continue
            inner = frag + bytes([content_type])
            if self.pad_to and content_type == CT_APPDATA:
                inner += b"\0" * min((-len(inner)) % self.pad_to, MAX_FRAGMENT + 1 - len(inner))
            hdr = struct.pack(">BHH", CT_APPDATA, 0x0303, len(inner) + 16)
            nonce = Tls13KeySchedule.record_nonce(self.write_key[1], self.write_seq)
            out += hdr + _aead_seal(self.suite, self.write_key[0], nonce, inner, hdr)
            self.write_seq += 1
        return bytes(out)

    def feed(self, data: bytes):
        """Yields the complete records in the bytes received so far as (content type, plaintext), one at a time: the
        caller handles each before the next is opened, because a handshake message may install new keys."""
        self.inbuf += data
        while len(self.inbuf) >= 5:
            ctype, version, n = struct.unpack(">BHH", self.inbuf[:5])
            if ctype not in (CT_CCS, CT_ALERT, CT_HANDSHAKE, CT_APPDATA) or version >> 8 != 3:
                raise TlsError("not a TLS record", ALERT_DECODE_ERROR)
            if n > MAX_FRAGMENT + 256:
                raise TlsError("record longer than the protocol allows", 22)              # record_overflow
            if len(self.inbuf) < 5 + n:
                break
            hdr, body = bytes(self.inbuf[:5]), bytes(self.inbuf[5:5 + n])
            del self.inbuf[:5 + n]
            if ctype == CT_CCS:
                if body != b"\x01":
                    raise TlsError("malformed ChangeCipherSpec", ALERT_UNEXPECTED_MESSAGE)
                continue                                                               # compatibility mode: ignored
            if self.read_key is not None:
                if ctype != CT_APPDATA:
                    raise TlsError("unprotected record after keys were installed", ALERT_UNEXPECTED_MESSAGE)
                nonce = Tls13KeySchedule.record_nonce(self.read_key[1], self.read_seq)
                inner = _aead_open(self.suite, self.read_key[0], nonce, body, hdr).rstrip(b"\0")
                self.read_seq += 1
                if not inner:
                    raise TlsError("record without a content type", ALERT_UNEXPECTED_MESSAGE)
                ctype, body = inner[-1], inner[:-1]
                if len(body) > MAX_FRAGMENT:
                    raise TlsError("record longer than the protocol allows", 22)
            elif ctype == CT_APPDATA:
                raise TlsError("protected record before any keys", ALERT_UNEXPECTED_MESSAGE)
            yield ctype, body


# -------------------------------------------------------------------------------------------------------- shared machinery
class Session:
    """What a client keeps from a NewSessionTicket to resume later."""

    def __init__(self, ticket: bytes, psk: bytes, suite: int, age_add: int, lifetime: int, issued: float):
        self.ticket, self.psk, self.suite, self.age_add, self.lifetime, self.issued = ticket, psk, suite, age_add, lifetime, issued

    def usable(self, now: Optional[float] = None) -> bool:
        return (time.time() if now is None else now) - self.issued < self.lifetime


class _Connection:
    """The parts both roles share: record layer, handshake reassembly, transcript, alerts, application data, KeyUpdate."""

    is_client = False

    def __init__(self, quic_transport_parameters: Optional[bytes] = None):
        self.records = _RecordLayer()
        # QUIC carries the handshake messages itself (RFC 9001 section 4): no records, no ChangeCipherSpec, no KeyUpdate
        # message; messages leave through ``crypto_out`` per encryption level and traffic secrets are handed over raw
        self.quic = quic_transport_parameters is not None
        self.quic_parameters = quic_transport_parameters
        self.peer_quic_parameters: Optional[bytes] = None
        self.crypto_out: Dict[str, bytearray] = {"initial": bytearray(), "handshake": bytearray(), "application": bytearray()}
        self.quic_secrets: Dict[Tuple[str, str], bytes] = {}          # (level, "read" | "write") -> traffic secret
        self._write_level = self._read_level = "initial"
        self.ks: Optional[Tls13KeySchedule] = None
        self.suite: Optional[int] = None
        self.transcript = hashlib.sha256()
        self.hs_buf = bytearray()
        self.out = bytearray()
        self.app_in = bytearray()
        self.handshake_complete = False
        self.closed = self.peer_closed = False
        self.used_psk = False
        self.alpn: Optional[str] = None
        self.peer_public_key: Optional[bytes] = None
        self.key_updates_sent = self.key_updates_received = 0

    # --- what the application calls
    def data_to_send(self) -> bytes:
        out = bytes(self.out)
        self.out.clear()
        return out

    def send(self, data: bytes) -> None:
        if not self.handshake_complete or self.closed:
            raise TlsError("connection is not open for application data")
        self.out += self.records.seal(CT_APPDATA, data)

    def read(self) -> bytes:
        out = bytes(self.app_in)
        self.app_in.clear()
        return out

    def close(self) -> None:
        if not self.closed:
            self.closed = True
            self.out += self.records.seal(CT_ALERT, bytes([1, ALERT_CLOSE_NOTIFY]))

    def update_keys(self, request_peer: bool = True) -> None:
        """Send KeyUpdate and move the sending direction to its next traffic secret (RFC 8446 section 4.6.3)."""
        if not self.handshake_complete or self.quic:
            raise TlsError("KeyUpdate before the handshake finished, or on a QUIC connection (which updates keys itself)")
        self.out += self.records.seal(CT_HANDSHAKE, _handshake(HS_KEY_UPDATE, bytes([1 if request_peer else 0])))
        label = "c ap traffic" if self.is_client else "s ap traffic"
        self.ks.update_traffic_secret(label)
        self._install_write(label)
        self.key_updates_sent += 1

    def export_keying_material(self, label: str, context: bytes = b"", length: int = 32) -> bytes:
        return self.ks.export_keying_material(label, context, length)

    def receive(self, data: bytes) -> None:
        """Feed bytes from the peer. Anything to answer with is in ``data_to_send()``; a fatal problem queues the alert
        and raises ``TlsError``."""
        try:
            for ctype, body in self.records.feed(data):
                if ctype == CT_ALERT:
                    self._on_alert(body)
                elif ctype == CT_HANDSHAKE:
                    self.hs_buf += body
                    self._drain_handshake()
                elif ctype == CT_APPDATA:
                    if not self.handshake_complete:
                        raise TlsError("application data during the handshake", ALERT_UNEXPECTED_MESSAGE)
                    if self.hs_buf:
                        raise TlsError("application data inside a handshake message", ALERT_UNEXPECTED_MESSAGE)
                    self.app_in += body
        except TlsError as e:
            if not e.received and not self.closed:
                self.closed = True
                self.out += self.records.seal(CT_ALERT, bytes([2, e.alert]))
            raise

    # --- internals
    def _on_alert(self, body: bytes) -> None:
        if len(body) != 2:
            raise TlsError("malformed alert", ALERT_DECODE_ERROR)
        if body[1] == ALERT_CLOSE_NOTIFY:
            self.peer_closed = True
            return
        self.closed = self.peer_closed = True
        raise TlsError(f"peer sent alert {body[1]}", body[1], received=True)

    def _drain_handshake(self) -> None:
        while len(self.hs_buf) >= 4:
            n = int.from_bytes(self.hs_buf[1:4], "big")
            if len(self.hs_buf) < 4 + n:
                return
            raw = bytes(self.hs_buf[:4 + n])
            del self.hs_buf[:4 + n]
            if self.handshake_complete:
                self._post_handshake(raw[0], raw[4:], raw)
            else:
                self._on_handshake(raw[0], raw[4:], raw)

    def _boundary(self) -> None:
        if self.hs_buf:
            raise TlsError("key change in the middle of a handshake message", ALERT_UNEXPECTED_MESSAGE)

    def _send_handshake(self, msg: bytes, in_transcript: bool = True) -> None:
        if in_transcript:
            self.transcript.update(msg)
        if self.quic:
            self.crypto_out[self._write_level] += msg
        else:
            self.out += self.records.seal(CT_HANDSHAKE, msg)

    @staticmethod
    def _level(label: str) -> str:
        return "handshake" if " hs " in label else "application"

    def _install_read(self, label: str) -> None:
        if self.quic:
            self._read_level = self._level(label)
            self.quic_secrets[(self._read_level, "read")] = self.ks.secrets[label]
        else:
            self.records.set_read(self.suite, self.ks.traffic_keys(label))

    def _install_write(self, label: str) -> None:
        if self.quic:
            self._write_level = self._level(label)
            self.quic_secrets[(self._write_level, "write")] = self.ks.secrets[label]
        else:
            self.records.set_write(self.suite, self.ks.traffic_keys(label))

    def receive_crypto(self, level: str, data: bytes) -> None:
        """QUIC mode: in-order bytes of the CRYPTO stream of one encryption level."""
        if not self.quic:
            raise TlsError("not a QUIC connection")
        if level != self._read_level:
            if data:
                raise TlsError(f"handshake data at level {level} while reading {self._read_level}", ALERT_UNEXPECTED_MESSAGE)
            return
        self.hs_buf += data
        self._drain_handshake()

    def _on_key_update(self, body: bytes) -> None:
        if self.quic:
            raise TlsError("KeyUpdate message on a QUIC connection", ALERT_UNEXPECTED_MESSAGE)
        if body not in (b"\0", b"\x01"):
            raise TlsError("malformed KeyUpdate", ALERT_ILLEGAL_PARAMETER)
        self._boundary()
        label = "s ap traffic" if self.is_client else "c ap traffic"
        self.ks.update_traffic_secret(label)
        self._install_read(label)
        self.key_updates_received += 1
        if body == b"\x01":
            self.update_keys(request_peer=False)

    def _on_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        raise NotImplementedError

    def _post_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        raise NotImplementedError


def _certificate_verify_input(transcript_hash: bytes, server: bool = True) -> bytes:
    who = b"TLS 1.3, server CertificateVerify" if server else b"TLS 1.3, client CertificateVerify"
    return b" " * 64 + who + b"\0" + transcript_hash


# ------------------------------------------------------------------------------------------------------------------ client
class TlsClient(_Connection):
    """Client side. ``start()`` queues the ClientHello; then alternate ``receive(bytes from the socket)`` and
    ``data_to_send()`` until ``handshake_complete``.

    Server authentication, at least one of: ``trusted_roots`` (DER certificates; the chain must reach one and cover
    ``server_name``), ``pinned_keys`` (accepted Ed25519 public keys of the leaf), ``psk`` = (identity, key) for an
    external pre-shared key, ``session`` from an earlier connection's ``sessions`` list. With a PSK or session the
    server may still fall back to a certificate handshake, which then has to pass the certificate checks."""

    is_client = True

    def __init__(self, server_name: Optional[str] = None, trusted_roots: Sequence[bytes] = (), pinned_keys: Iterable[bytes] = (),
                 psk: Optional[Tuple[bytes, bytes]] = None, session: Optional[Session] = None, alpn: Sequence[str] = (),
                 suites: Sequence[int] = SUITES, insecure_skip_verify: bool = False,
                 quic_transport_parameters: Optional[bytes] = None):
        super().__init__(quic_transport_parameters)
        if self.quic and not alpn:
            raise ValueError("QUIC requires an application protocol to be negotiated")
        self.server_name, self.trusted_roots, self.pinned_keys = server_name, list(trusted_roots), set(pinned_keys)
        self.psk, self.session, self.alpn_offer, self.suites = psk, session, list(alpn), list(suites)
        self.skip_verify = insecure_skip_verify
        if session is not None and psk is not None:
            raise ValueError("offer either an external PSK or a session, not both")
        if not (self.trusted_roots or self.pinned_keys or psk or session or insecure_skip_verify):
            raise ValueError("no way to authenticate the server: give trusted_roots, pinned_keys, psk or session")
        self.sessions: List[Session] = []
        self._private = os.urandom(32)
        self._state = "start"
        self._server_chain: List[bytes] = []
        self._psk_key: Optional[bytes] = None

    def start(self) -> None:
        if self._state != "start":
            raise TlsError("handshake already started")
        exts: List[Tuple[int, bytes]] = []
        if self.server_name:
            exts.append((EXT_SERVER_NAME, _v16(b"\0" + _v16(self.server_name.encode()))))
        exts += [(EXT_SUPPORTED_VERSIONS, _v8(b"\x03\x04")), (EXT_SUPPORTED_GROUPS, _v16(struct.pack(">H", GROUP_X25519))),
                 (EXT_SIGNATURE_ALGORITHMS, _v16(struct.pack(">H", SIG_ED25519))),
                 (EXT_KEY_SHARE, _v16(struct.pack(">H", GROUP_X25519) + _v16(crypto.x25519(self._private))))]
        if self.alpn_offer:
            exts.append((EXT_ALPN, _v16(b"".join(_v8(p.encode()) for p in self.alpn_offer))))
        if self.quic:
            exts.append((EXT_QUIC_TRANSPORT_PARAMETERS, self.quic_parameters))
        identity, age, external = None, 0, True
        if self.psk is not None:
            identity, self._psk_key = self.psk
        elif self.session is not None and self.session.usable():
            identity, self._psk_key, external = self.session.ticket, self.session.psk, False
            age = (int((time.time() - self.session.issued) * 1000) + self.session.age_add) & 0xFFFFFFFF
            self.suites = [self.session.suite] + [s for s in self.suites if s != self.session.suite]
        if identity is not None:
            exts.append((EXT_PSK_MODES, _v8(bytes([PSK_DHE_KE]))))
            exts.append((EXT_PRE_SHARED_KEY, _v16(_v16(identity) + struct.pack(">I", age)) + _v16(_v8(b"\0" * 32))))
        self._session_id = b"" if self.quic else os.urandom(32)        # QUIC does not use compatibility mode
        body = b"\x03\x03" + os.urandom(32) + _v8(self._session_id) + _v16(b"".join(struct.pack(">H", s) for s in self.suites)) \
            + _v8(b"\0") + _extensions(exts)
        hello = _handshake(HS_CLIENT_HELLO, body)
        if identity is not None:                          # the binder covers the hello up to the binders list (2 + 1 + 32 bytes)
            early = Tls13KeySchedule(self.suites[0], self._psk_key)
            fk = hkdf_expand_label(early.binder_key(external), "finished", b"", 32)
            binder = crypto.hmac_sha256(fk, hashlib.sha256(hello[:-35]).digest())
            hello = hello[:-32] + binder
        self._send_handshake(hello)
        self._state = "wait_server_hello"

    def _on_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        handler = {"wait_server_hello": self._server_hello, "wait_encrypted_extensions": self._encrypted_extensions,
                   "wait_certificate": self._certificate, "wait_certificate_verify": self._certificate_verify,
                   "wait_finished": self._finished}.get(self._state)
        if handler is None:
            raise TlsError(f"handshake message {msg_type} in state {self._state}", ALERT_UNEXPECTED_MESSAGE)
        handler(msg_type, body, raw)

    def _server_hello(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type != HS_SERVER_HELLO:
            raise TlsError("expected ServerHello", ALERT_UNEXPECTED_MESSAGE)
        r = _Reader(body)
        legacy_version, random, session_id, suite, compression = r.take(2), r.take(32), r.vec(1), r.u16(), r.u8()
        ext = _parse_extensions(r)
        if random == HRR_RANDOM:
            raise TlsError("HelloRetryRequest is not supported", ALERT_HANDSHAKE_FAILURE)
        if legacy_version != b"\x03\x03" or ext.get(EXT_SUPPORTED_VERSIONS) != b"\x03\x04":
            raise TlsError("server did not negotiate TLS 1.3", ALERT_PROTOCOL_VERSION)
        if session_id != self._session_id or compression != 0 or suite not in self.suites:
            raise TlsError("ServerHello does not answer this ClientHello", ALERT_ILLEGAL_PARAMETER)
        if EXT_KEY_SHARE not in ext:
            raise TlsError("ServerHello without a key share", ALERT_MISSING_EXTENSION)
        kr = _Reader(ext[EXT_KEY_SHARE])
        group, share = kr.u16(), kr.vec(2)
        if group != GROUP_X25519 or len(share) != 32:
            raise TlsError("server chose a group that was not offered", ALERT_ILLEGAL_PARAMETER)
        if EXT_PRE_SHARED_KEY in ext:
            if self._psk_key is None or ext[EXT_PRE_SHARED_KEY] != b"\0\0":
                raise TlsError("server selected a PSK that was not offered", ALERT_ILLEGAL_PARAMETER)
            if self.session is not None and suite != self.session.suite and self.psk is None:
                raise TlsError("resumed with a different hash", ALERT_ILLEGAL_PARAMETER)
            self.used_psk = True
        self.suite = suite
        self.ks = Tls13KeySchedule(suite, self._psk_key if self.used_psk else None)
        shared = crypto.x25519(self._private, share)
        if shared == b"\0" * 32:
            raise TlsError("key share of small order", ALERT_ILLEGAL_PARAMETER)
        self.transcript.update(raw)
        self.ks.set_shared_secret(shared, self.transcript.digest())
        self._boundary()
        self._install_read("s hs traffic")
        self._state = "wait_encrypted_extensions"

    def _encrypted_extensions(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type != HS_ENCRYPTED_EXTENSIONS:
            raise TlsError("expected EncryptedExtensions", ALERT_UNEXPECTED_MESSAGE)
        ext = _parse_extensions(_Reader(body))
        if EXT_ALPN in ext:
            names = _Reader(_Reader(ext[EXT_ALPN]).vec(2))
            chosen = names.vec(1).decode()
            if chosen not in self.alpn_offer or not names.done():
                raise TlsError("server chose a protocol that was not offered", ALERT_ILLEGAL_PARAMETER)
            self.alpn = chosen
        if self.quic:
            if EXT_QUIC_TRANSPORT_PARAMETERS not in ext:
                raise TlsError("server sent no QUIC transport parameters", ALERT_MISSING_EXTENSION)
            if self.alpn is None:
                raise TlsError("server chose no application protocol", ALERT_NO_APPLICATION_PROTOCOL)
            self.peer_quic_parameters = ext[EXT_QUIC_TRANSPORT_PARAMETERS]
        self.transcript.update(raw)
        self._state = "wait_finished" if self.used_psk else "wait_certificate"

    def _certificate(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type == HS_CERTIFICATE_REQUEST:
            raise TlsError("client certificates are not supported", ALERT_HANDSHAKE_FAILURE)
        if msg_type != HS_CERTIFICATE:
            raise TlsError("expected Certificate", ALERT_UNEXPECTED_MESSAGE)
        r = _Reader(body)
        if r.vec(1) != b"":
            raise TlsError("server certificate with a request context", ALERT_ILLEGAL_PARAMETER)
        entries = _Reader(r.vec(3))
        while not entries.done():
            self._server_chain.append(entries.vec(3))
            entries.vec(2)                                                                 # per-certificate extensions
        if not self._server_chain:
            raise TlsError("empty certificate list", ALERT_DECODE_ERROR)
        self.transcript.update(raw)
        self._state = "wait_certificate_verify"

    def _certificate_verify(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type != HS_CERTIFICATE_VERIFY:
            raise TlsError("expected CertificateVerify", ALERT_UNEXPECTED_MESSAGE)
        r = _Reader(body)
        scheme, signature = r.u16(), r.vec(2)
        if scheme != SIG_ED25519:
            raise TlsError("signature scheme that was not offered", ALERT_ILLEGAL_PARAMETER)
        try:
            leaf = parse_certificate(self._server_chain[0])
        except (ValueError, IndexError) as e:
            raise TlsError(f"unreadable certificate: {e}", ALERT_BAD_CERTIFICATE) from e
        if leaf["key_oid"] != OID_ED25519:
            raise TlsError("only Ed25519 certificates are supported", ALERT_BAD_CERTIFICATE)
        if not crypto.ed25519_verify(leaf["public_key"], _certificate_verify_input(self.transcript.digest()), signature):
            raise TlsError("CertificateVerify does not verify", ALERT_DECRYPT_ERROR)
        if leaf["public_key"] in self.pinned_keys or self.skip_verify:
            pass
        elif self.trusted_roots:
            verify_chain(self._server_chain, self.trusted_roots, self.server_name)
        else:
            raise TlsError("server fell back to a certificate and nothing is configured to check it", ALERT_BAD_CERTIFICATE)
        self.peer_public_key = leaf["public_key"]
        self.transcript.update(raw)
        self._state = "wait_finished"

    def _finished(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type != HS_FINISHED:
            raise TlsError("expected Finished", ALERT_UNEXPECTED_MESSAGE)
        if not self.ks.verify_finished("s hs traffic", self.transcript.digest(), body):
            raise TlsError("server Finished does not verify", ALERT_DECRYPT_ERROR)
        self.transcript.update(raw)
        self._boundary()
        self.ks.set_server_finished(self.transcript.digest())
        if not self.quic:
            self.out += self.records.seal(CT_CCS, b"\x01")                                 # compatibility mode
        self._install_write("c hs traffic")
        self._send_handshake(_handshake(HS_FINISHED, self.ks.finished_mac("c hs traffic", self.transcript.digest())))
        self.ks.set_client_finished(self.transcript.digest())
        self._install_read("s ap traffic")
        self._install_write("c ap traffic")
        self.handshake_complete, self._state = True, "connected"

    def _post_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type == HS_KEY_UPDATE:
            self._on_key_update(body)
        elif msg_type == HS_NEW_SESSION_TICKET:
            r = _Reader(body)
            lifetime, age_add, nonce, ticket = r.u32(), r.u32(), r.vec(1), r.vec(2)
            _parse_extensions(r)
            if lifetime > 0 and ticket:
                self.sessions.append(Session(ticket, self.ks.resumption_psk(nonce), self.suite, age_add, min(lifetime, 604800),
                                             time.time()))
        else:
            raise TlsError(f"handshake message {msg_type} after the handshake", ALERT_UNEXPECTED_MESSAGE)


# ------------------------------------------------------------------------------------------------------------------ server
class TicketStore:
    """Server-side session state for resumption: tickets are random handles to entries kept here (single use)."""

    def __init__(self, lifetime: int = 7200, capacity: int = 4096):
        self.lifetime, self.capacity = lifetime, capacity
        self._entries: Dict[bytes, Tuple[bytes, int, int, float]] = {}

    def issue(self, psk: bytes, suite: int) -> Tuple[bytes, int]:
        if len(self._entries) >= self.capacity:
            self._entries.pop(next(iter(self._entries)))
        ticket, age_add = os.urandom(32), int.from_bytes(os.urandom(4), "big")
        self._entries[ticket] = (psk, suite, age_add, time.time())
        return ticket, age_add

    def redeem(self, ticket: bytes, obfuscated_age: int, tolerance_ms: int = 10000) -> Optional[Tuple[bytes, int]]:
        entry = self._entries.get(ticket)
        if entry is None:
            return None
        psk, suite, age_add, issued = entry
        real_ms = (time.time() - issued) * 1000
        claimed_ms = (obfuscated_age - age_add) & 0xFFFFFFFF
        if real_ms > self.lifetime * 1000 or abs(real_ms - claimed_ms) > tolerance_ms:
            self._entries.pop(ticket, None)
            return None
        return psk, suite

    def consume(self, ticket: bytes) -> None:
        self._entries.pop(ticket, None)


class TlsServer(_Connection):
    """Server side of one connection. ``certificate_chain`` (DER, leaf first) with ``private_seed`` (the leaf's Ed25519
    seed) enables certificate handshakes; ``psk_lookup(identity) -> key or None`` enables external PSKs; ``tickets``
    (shared between the connections of one listener) enables resumption, ``send_tickets`` of them per connection."""

    def __init__(self, certificate_chain: Sequence[bytes] = (), private_seed: Optional[bytes] = None,
                 psk_lookup: Optional[Callable[[bytes], Optional[bytes]]] = None, tickets: Optional[TicketStore] = None,
                 alpn: Sequence[str] = (), suites: Sequence[int] = SUITES, send_tickets: int = 1,
                 quic_transport_parameters: Optional[bytes] = None):
        super().__init__(quic_transport_parameters)
        if self.quic and not alpn:
            raise ValueError("QUIC requires an application protocol to be negotiated")
        if bool(certificate_chain) != bool(private_seed):
            raise ValueError("a certificate chain needs its private seed, and the other way round")
        if not certificate_chain and psk_lookup is None:
            raise ValueError("nothing to authenticate with: give a certificate or a PSK lookup")
        self.chain, self.seed, self.psk_lookup, self.tickets = list(certificate_chain), private_seed, psk_lookup, tickets
        self.alpn_supported, self.suites, self.send_tickets = list(alpn), list(suites), send_tickets
        self._state = "wait_client_hello"
        self.server_name: Optional[str] = None
        self.psk_identity: Optional[bytes] = None
        self.resumed = False

    def _on_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if self._state == "wait_client_hello" and msg_type == HS_CLIENT_HELLO:
            self._client_hello(body, raw)
        elif self._state == "wait_finished" and msg_type == HS_FINISHED:
            self._client_finished(body, raw)
        else:
            raise TlsError(f"handshake message {msg_type} in state {self._state}", ALERT_UNEXPECTED_MESSAGE)

    def _select_psk(self, ext: Dict[int, bytes], raw: bytes) -> Optional[Tuple[int, bytes, Optional[int]]]:
        """(index, key, suite the ticket was issued under or None) of the first offered identity that is known and whose
        binder verifies; a known identity with a wrong binder is fatal."""
        if EXT_PRE_SHARED_KEY not in ext:
            return None
        modes = _Reader(ext.get(EXT_PSK_MODES, b"\0")).vec(1)
        r = _Reader(ext[EXT_PRE_SHARED_KEY])
        ids, binders = _Reader(r.vec(2)), _Reader(r.vec(2))
        binders_len = 2 + len(binders.buf)
        if not raw.endswith(ext[EXT_PRE_SHARED_KEY]):
            raise TlsError("pre_shared_key is not the last extension", ALERT_ILLEGAL_PARAMETER)
        offered, blist = [], []
        while not ids.done():
            offered.append((ids.vec(2), ids.u32()))
        while not binders.done():
            blist.append(binders.vec(1))
        if len(offered) != len(blist) or not offered:
            raise TlsError("identities and binders do not pair up", ALERT_ILLEGAL_PARAMETER)
        if PSK_DHE_KE not in modes:
            return None
        truncated = hashlib.sha256(raw[:-binders_len]).digest()
        for i, (identity, age) in enumerate(offered):
            key, external, ticket_suite = None, True, None
            if self.tickets is not None:
                hit = self.tickets.redeem(identity, age)
                if hit is not None:
                    key, ticket_suite = hit
                    external = False
            if key is None and self.psk_lookup is not None:
                key = self.psk_lookup(identity)
            if key is None:
                continue
            fk = hkdf_expand_label(Tls13KeySchedule(self.suites[0], key).binder_key(external), "finished", b"", 32)
            if not crypto.ct_equal(crypto.hmac_sha256(fk, truncated), blist[i]):
                raise TlsError("PSK binder does not verify", ALERT_DECRYPT_ERROR)
            if not external:
                self.tickets.consume(identity)
                self.resumed = True
            self.psk_identity = identity
            return i, key, ticket_suite
        return None

    def _client_hello(self, body: bytes, raw: bytes) -> None:
        r = _Reader(body)
        r.take(2), r.take(32)
        session_id, suites_raw, compression = r.vec(1), r.vec(2), r.vec(1)
        ext = _parse_extensions(r)
        versions = ext.get(EXT_SUPPORTED_VERSIONS, b"")
        if b"\x03\x04" not in [versions[i:i + 2] for i in range(1, len(versions), 2)]:
            raise TlsError("client does not offer TLS 1.3", ALERT_PROTOCOL_VERSION)
        if compression != b"\0" or len(session_id) > 32:
            raise TlsError("malformed ClientHello", ALERT_ILLEGAL_PARAMETER)
        offered = [struct.unpack(">H", suites_raw[i:i + 2])[0] for i in range(0, len(suites_raw) - 1, 2)]
        if EXT_SERVER_NAME in ext:
            sr = _Reader(_Reader(ext[EXT_SERVER_NAME]).vec(2))
            if sr.u8() == 0:
                self.server_name = sr.vec(2).decode(errors="replace")
        share = None
        if EXT_KEY_SHARE in ext:
            kr = _Reader(_Reader(ext[EXT_KEY_SHARE]).vec(2))
            while not kr.done():
                group, key = kr.u16(), kr.vec(2)
                if group == GROUP_X25519 and len(key) == 32:
                    share = key
        if share is None:
            raise TlsError("no x25519 key share (HelloRetryRequest is not supported)", ALERT_HANDSHAKE_FAILURE)
        psk = self._select_psk(ext, raw)
        suite = next((s for s in self.suites if s in offered), None)
        if psk is not None and psk[2] is not None and psk[2] in offered:
            suite = psk[2]
        if suite is None:
            raise TlsError("no cipher suite in common", ALERT_HANDSHAKE_FAILURE)
        if psk is None:
            if not self.chain:
                raise TlsError("no PSK identity matched and there is no certificate", ALERT_UNKNOWN_PSK_IDENTITY)
            sigs = _Reader(ext.get(EXT_SIGNATURE_ALGORITHMS, b"\0\0")).vec(2)
            if struct.pack(">H", SIG_ED25519) not in [sigs[i:i + 2] for i in range(0, len(sigs), 2)]:
                raise TlsError("client does not accept ed25519 signatures", ALERT_HANDSHAKE_FAILURE)
        if EXT_ALPN in ext and self.alpn_supported:
            names, theirs = _Reader(_Reader(ext[EXT_ALPN]).vec(2)), []
            while not names.done():
                theirs.append(names.vec(1).decode(errors="replace"))
            self.alpn = next((p for p in self.alpn_supported if p in theirs), None)
            if self.alpn is None:
                raise TlsError("no application protocol in common", ALERT_NO_APPLICATION_PROTOCOL)
        if self.quic:
            if EXT_QUIC_TRANSPORT_PARAMETERS not in ext:
                raise TlsError("client sent no QUIC transport parameters", ALERT_MISSING_EXTENSION)
            if self.alpn is None:
                raise TlsError("no application protocol in common", ALERT_NO_APPLICATION_PROTOCOL)
            self.peer_quic_parameters = ext[EXT_QUIC_TRANSPORT_PARAMETERS]
        self.suite, self.used_psk = suite, psk is not None
        self.ks = Tls13KeySchedule(suite, psk[1] if psk else None)
        self.transcript.update(raw)
        private = os.urandom(32)
        shared = crypto.x25519(private, share)
        if shared == b"\0" * 32:
            raise TlsError("key share of small order", ALERT_ILLEGAL_PARAMETER)
        sh_ext = [(EXT_SUPPORTED_VERSIONS, b"\x03\x04"), (EXT_KEY_SHARE, struct.pack(">H", GROUP_X25519) + _v16(crypto.x25519(private)))]
        if psk is not None:
            sh_ext.append((EXT_PRE_SHARED_KEY, struct.pack(">H", psk[0])))
        self._send_handshake(_handshake(HS_SERVER_HELLO, b"\x03\x03" + os.urandom(32) + _v8(session_id) + struct.pack(">H", suite)
                                        + b"\0" + _extensions(sh_ext)))
        if not self.quic:
            self.out += self.records.seal(CT_CCS, b"\x01")
        self.ks.set_shared_secret(shared, self.transcript.digest())
        self._install_write("s hs traffic")
        ee = [(EXT_ALPN, _v16(_v8(self.alpn.encode())))] if self.alpn else []
        if self.quic:
            ee.append((EXT_QUIC_TRANSPORT_PARAMETERS, self.quic_parameters))
        self._send_handshake(_handshake(HS_ENCRYPTED_EXTENSIONS, _extensions(ee)))
        if psk is None:
            certs = b"".join(_v24(c) + _v16(b"") for c in self.chain)
            self._send_handshake(_handshake(HS_CERTIFICATE, _v8(b"") + _v24(certs)))
            sig = crypto.ed25519_sign(self.seed, _certificate_verify_input(self.transcript.digest()))
            self._send_handshake(_handshake(HS_CERTIFICATE_VERIFY, struct.pack(">H", SIG_ED25519) + _v16(sig)))
        self._send_handshake(_handshake(HS_FINISHED, self.ks.finished_mac("s hs traffic", self.transcript.digest())))
        self.ks.set_server_finished(self.transcript.digest())
        self._install_write("s ap traffic")
        self._boundary()
        self._install_read("c hs traffic")
        self._state = "wait_finished"

    def _client_finished(self, body: bytes, raw: bytes) -> None:
        if not self.ks.verify_finished("c hs traffic", self.transcript.digest(), body):
            raise TlsError("client Finished does not verify", ALERT_DECRYPT_ERROR)
        self.transcript.update(raw)
        self._boundary()
        self.ks.set_client_finished(self.transcript.digest())
        self._install_read("c ap traffic")
        self.handshake_complete, self._state = True, "connected"
        if self.tickets is not None:
            for i in range(self.send_tickets):
                nonce = bytes([i])
                ticket, age_add = self.tickets.issue(self.ks.resumption_psk(nonce), self.suite)
                msg = struct.pack(">II", self.tickets.lifetime, age_add) + _v8(nonce) + _v16(ticket) + _extensions([])
                self._send_handshake(_handshake(HS_NEW_SESSION_TICKET, msg), in_transcript=False)

    def _post_handshake(self, msg_type: int, body: bytes, raw: bytes) -> None:
        if msg_type != HS_KEY_UPDATE:
            raise TlsError(f"handshake message {msg_type} after the handshake", ALERT_UNEXPECTED_MESSAGE)
        self._on_key_update(body)


# ----------------------------------------------------------------------------------------------------------------- sockets
class TlsSocket:
    """A connected TCP socket driven through a ``TlsClient`` or ``TlsServer``: blocking ``handshake``, ``sendall``,
    ``recv``, ``close``."""

    def __init__(self, sock: socket.socket, connection: _Connection):
        self.sock, self.conn = sock, connection

    def _flush(self) -> None:
        data = self.conn.data_to_send()
        if data:
            self.sock.sendall(data)

    def _pump(self) -> bool:
        data = self.sock.recv(65536)
        if not data:
            return False
        try:
            self.conn.receive(data)
        finally:
            self._flush()
        return True

    def handshake(self) -> "TlsSocket":
        if self.conn.is_client:
            self.conn.start()
        self._flush()
        while not self.conn.handshake_complete:
            if not self._pump():
                raise TlsError("connection closed during the handshake", ALERT_UNEXPECTED_MESSAGE)
        return self

    def sendall(self, data: bytes) -> None:
        self.conn.send(data)
        self._flush()

    def recv(self) -> bytes:
        """The next application bytes; b"" once the peer has closed."""
        while True:
            data = self.conn.read()
            if data or self.conn.peer_closed:
                return data
            if not self._pump():
                return self.conn.read()

    def close(self) -> None:
        try:
            self.conn.close()
            self._flush()
        except OSError:
            pass
        finally:
            self.sock.close()


def connect(address: Tuple[str, int], timeout: float = 10.0, **client_options) -> TlsSocket:
    """Open a TCP connection and complete a handshake as a client; options as for ``TlsClient``."""
    sock = socket.create_connection(address, timeout=timeout)
    try:
        return TlsSocket(sock, TlsClient(**client_options)).handshake()
    except BaseException:
        sock.close()
        raise
