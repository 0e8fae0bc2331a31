"""S4 extensions: protocol pieces and packet-level defences around the serving and cluster endpoints.

* ``Tls13KeySchedule``: the RFC 8446 section 7.1 key schedule on SHA-256 (early / handshake / master secrets,
  traffic secrets and keys, Finished MACs, exporters, key update) and cipher-suite negotiation;
* ``NoiseHandshake``: the Noise protocol framework (revision 34) for patterns NN, NK, XX and IK over X25519,
  ChaCha20-Poly1305 and SHA-256, with ``split`` into two transport ``CipherState`` s;
* ``TunnelPeer``: a WireGuard-shaped tunnel on Noise IK: counters with a sliding replay window, rekey limits,
  keep-alives, per-peer byte counters;
* ``IPBlocklist`` (CIDR trie, v4 and v6), ``Nids`` (header parsing, scan / flag anomalies, content rules in a
  Snort-like syntax), traffic padding and fragmentation, ``PortKnock`` (time-windowed knock sequences),
  ``GrpcAuth`` (rotating bearer metadata), ``DohResolver`` (RFC 8484 wire format, TTL cache), certificate
  transparency (RFC 6962 Merkle inclusion / consistency proofs, SCT parsing and signature check).

Reference behaviour: security/network/s4_extensions.c (function families ``tls13_*``, ``noise_*``, ``wireguard_*``,
``ip_blocklist_*``, ``nids_*``, ``traffic_pad*``, ``port_knock_*``, ``grpc_auth_*``, ``doh_*``, ``ct_verify_*``).
Rate limiting, OCSP caching and the QUIC-shaped transport are in ``security/network.py``, ``security/services.py`` and
``utils/quic.py``.
"""
from __future__ import annotations

import base64
import hashlib
import hmac as _hmac
import ipaddress
import os
import re
import struct
import time
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from . import crypto


# ------------------------------------------------------------------------------------------------ TLS 1.3 key schedule
TLS_AES_128_GCM_SHA256, TLS_AES_256_GCM_SHA384, TLS_CHACHA20_POLY1305_SHA256 = 0x1301, 0x1302, 0x1303
_SUITE_KEY_LEN = {TLS_AES_128_GCM_SHA256: 16, TLS_CHACHA20_POLY1305_SHA256: 32}


def negotiate_cipher(client_suites: Sequence[int], server_preference: Sequence[int] = (TLS_CHACHA20_POLY1305_SHA256,
                                                                                         TLS_AES_128_GCM_SHA256)) -> Optional[int]:
    """First suite of the server's preference list that the client offers (SHA-256 suites only), or None."""
    offered = set(client_suites)
    return next((s for s in server_preference if s in offered and s in _SUITE_KEY_LEN), None)


def hkdf_extract(salt: bytes, ikm: bytes) -> bytes:
    return crypto.hmac_sha256(salt if salt else b"\0" * 32, ikm)


def hkdf_expand(prk: bytes, info: bytes, length: int) -> bytes:
    out, t, i = b"", b"", 1
    while len(out) < length:
        t = crypto.hmac_sha256(prk, t + info + bytes([i]))
        out, i = out + t, i + 1
    return out[:length]


def hkdf_expand_label(secret: bytes, label: str, context: bytes, length: int) -> bytes:
    full = b"tls13 " + label.encode()
    info = struct.pack(">H", length) + bytes([len(full)]) + full + bytes([len(context)]) + context
    return hkdf_expand(secret, info, length)


class Tls13KeySchedule:
    """Secrets of one TLS 1.3 connection. Feed it the PSK (or nothing), the (EC)DHE shared secret and the transcript
    hashes at the points RFC 8446 names; read traffic keys and Finished values back."""

    EMPTY_HASH = hashlib.sha256(b"").digest()

    def __init__(self, suite: int = TLS_CHACHA20_POLY1305_SHA256, psk: Optional[bytes] = None):
        if suite not in _SUITE_KEY_LEN:
            raise ValueError("only the SHA-256 cipher suites are supported")
        self.suite, self.key_len = suite, _SUITE_KEY_LEN[suite]
        self.early_secret = hkdf_extract(b"", psk if psk else b"\0" * 32)
        self.handshake_secret = self.master_secret = None
        self.secrets: Dict[str, bytes] = {}
        self.key_generation = 0

    def derive_secret(self, secret: bytes, label: str, transcript_hash: bytes) -> bytes:
        return hkdf_expand_label(secret, label, transcript_hash, 32)

    def binder_key(self, external: bool = True) -> bytes:
        return self.derive_secret(self.early_secret, "ext binder" if external else "res binder", self.EMPTY_HASH)

    def early_traffic(self, client_hello_hash: bytes) -> bytes:
        self.secrets["c e traffic"] = self.derive_secret(self.early_secret, "c e traffic", client_hello_hash)
        return self.secrets["c e traffic"]

    def set_shared_secret(self, dhe: bytes, hello_hash: bytes) -> None:
        """After ServerHello: handshake secret and both handshake traffic secrets (transcript = CH..SH)."""
        derived = self.derive_secret(self.early_secret, "derived", self.EMPTY_HASH)
        self.handshake_secret = hkdf_extract(derived, dhe)
        for lab in ("c hs traffic", "s hs traffic"):
            self.secrets[lab] = self.derive_secret(self.handshake_secret, lab, hello_hash)
        self.master_secret = hkdf_extract(self.derive_secret(self.handshake_secret, "derived", self.EMPTY_HASH), b"\0" * 32)

    def set_server_finished(self, transcript_hash: bytes) -> None:
        """After the server's Finished: application traffic secrets and the exporter master secret."""
        if self.master_secret is None:
            raise RuntimeError("the shared secret has not been set")
        for lab in ("c ap traffic", "s ap traffic", "exp master"):
            self.secrets[lab] = self.derive_secret(self.master_secret, lab, transcript_hash)

    def set_client_finished(self, transcript_hash: bytes) -> bytes:
        self.secrets["res master"] = self.derive_secret(self.master_secret, "res master", transcript_hash)
        return self.secrets["res master"]

    def traffic_keys(self, label: str) -> Tuple[bytes, bytes]:
        """(key, 12-byte IV) of a traffic secret such as "s hs traffic" or "c ap traffic"."""
        s = self.secrets[label]
        return hkdf_expand_label(s, "key", b"", self.key_len), hkdf_expand_label(s, "iv", b"", 12)

    def finished_mac(self, label: str, transcript_hash: bytes) -> bytes:
        return crypto.hmac_sha256(hkdf_expand_label(self.secrets[label], "finished", b"", 32), transcript_hash)

    def verify_finished(self, label: str, transcript_hash: bytes, received: bytes) -> bool:
        return _hmac.compare_digest(self.finished_mac(label, transcript_hash), received)

    def export_keying_material(self, label: str, context: bytes = b"", length: int = 32) -> bytes:
        s = self.derive_secret(self.secrets["exp master"], label, self.EMPTY_HASH)
        return hkdf_expand_label(s, "exporter", hashlib.sha256(context).digest(), length)

    def update_traffic_secret(self, label: str) -> bytes:
        """KeyUpdate: application_traffic_secret_N+1 = HKDF-Expand-Label(secret_N, "traffic upd", "", 32)."""
        self.secrets[label] = hkdf_expand_label(self.secrets[label], "traffic upd", b"", 32)
        self.key_generation += 1
        return self.secrets[label]

    def resumption_psk(self, ticket_nonce: bytes) -> bytes:
        return hkdf_expand_label(self.secrets["res master"], "resumption", ticket_nonce, 32)

    @staticmethod
    def record_nonce(iv: bytes, sequence: int) -> bytes:
        """Per-record nonce: the 64-bit record sequence number, left-padded, XORed into the static IV."""
        return bytes(a ^ b for a, b in zip(iv, sequence.to_bytes(12, "big")))


# ------------------------------------------------------------------------------------------------ Noise framework
class NoiseError(RuntimeError):
    pass


class CipherState:
    """ChaCha20-Poly1305 with a 64-bit counter nonce (4 zero bytes || little-endian counter)."""

    MAX_NONCE = 2 ** 64 - 1

    def __init__(self, key: Optional[bytes] = None):
        self.k, self.n = key, 0

    def has_key(self) -> bool:
        return self.k is not None

    def _nonce(self, n: int) -> bytes:
        return b"\0\0\0\0" + n.to_bytes(8, "little")

    def encrypt_with_ad(self, ad: bytes, plaintext: bytes) -> bytes:
        if self.k is None:
            return plaintext
        if self.n >= self.MAX_NONCE:
            raise NoiseError("nonce exhausted")
        out = crypto.aead_encrypt(self.k, self._nonce(self.n), plaintext, ad)
        self.n += 1
        return out

    def decrypt_with_ad(self, ad: bytes, ciphertext: bytes) -> bytes:
        if self.k is None:
            return ciphertext
        if self.n >= self.MAX_NONCE:
            raise NoiseError("nonce exhausted")
        try:
            out = crypto.aead_decrypt(self.k, self._nonce(self.n), ciphertext, ad)
        except ValueError as e:
            raise NoiseError("decryption failed") from e
        self.n += 1
        return out

    def decrypt_at(self, n: int, ad: bytes, ciphertext: bytes) -> bytes:
        """Decrypt with an explicit counter (transports that carry the counter in the packet)."""
        try:
            return crypto.aead_decrypt(self.k, self._nonce(n), ciphertext, ad)
        except ValueError as e:
            raise NoiseError("decryption failed") from e

    def rekey(self) -> None:
        self.k = crypto.aead_encrypt(self.k, self._nonce(self.MAX_NONCE), b"\0" * 32, b"")[:32]


class _SymmetricState:
    def __init__(self, protocol_name: bytes):
        self.h = protocol_name.ljust(32, b"\0") if len(protocol_name) <= 32 else crypto.sha256(protocol_name)
        self.ck = self.h
        self.cipher = CipherState()

    def mix_hash(self, data: bytes) -> None:
        self.h = crypto.sha256(self.h + data)

    def _hkdf2(self, ikm: bytes) -> Tuple[bytes, bytes]:
        temp = crypto.hmac_sha256(self.ck, ikm)
        o1 = crypto.hmac_sha256(temp, b"\x01")
        return o1, crypto.hmac_sha256(temp, o1 + b"\x02")

    def mix_key(self, ikm: bytes) -> None:
        self.ck, k = self._hkdf2(ikm)
        self.cipher = CipherState(k)

    def encrypt_and_hash(self, plaintext: bytes) -> bytes:
        ct = self.cipher.encrypt_with_ad(self.h, plaintext)
        self.mix_hash(ct)
        return ct

    def decrypt_and_hash(self, ciphertext: bytes) -> bytes:
        pt = self.cipher.decrypt_with_ad(self.h, ciphertext)
        self.mix_hash(ciphertext)
        return pt

    def split(self) -> Tuple[CipherState, CipherState]:
        k1, k2 = self._hkdf2(b"")
        return CipherState(k1), CipherState(k2)


# pattern: (initiator pre-message keys, responder pre-message keys, message token lists in order)
NOISE_PATTERNS = {
    "NN": ((), (), (("e",), ("e", "ee"))),
    "NK": ((), ("s",), (("e", "es"), ("e", "ee"))),
    "XX": ((), (), (("e",), ("e", "ee", "s", "es"), ("s", "se"))),
    "IK": ((), ("s",), (("e", "es", "s", "ss"), ("e", "ee", "se"))),
}


class NoiseHandshake:
    """One side of a Noise handshake. ``s`` is this side's static private key (needed when the pattern sends or
    pre-shares it), ``rs`` the peer's static public key when the pattern pre-shares it, ``e`` an ephemeral private key
    (random when omitted; fixed in tests). Alternate ``write_message`` / ``read_message`` in the pattern's order; after
    the last message ``split()`` gives (cipher for initiator->responder, cipher for responder->initiator)."""

    def __init__(self, pattern: str, initiator: bool, s: Optional[bytes] = None, rs: Optional[bytes] = None,
                 e: Optional[bytes] = None, prologue: bytes = b""):
        if pattern not in NOISE_PATTERNS:
            raise ValueError(f"unsupported Noise pattern {pattern!r}")
        self.pattern, self.initiator = pattern, initiator
        self.s, self.rs, self.e, self.re = s, rs, e, None
        pre_i, pre_r, self._messages = NOISE_PATTERNS[pattern]
        self._ss = _SymmetricState(f"Noise_{pattern}_25519_ChaChaPoly_SHA256".encode())
        self._ss.mix_hash(prologue)
        for who, toks in ((True, pre_i), (False, pre_r)):
            for _ in toks:                                   # only "s" occurs in the supported patterns
                pub = crypto.x25519(self.s) if who == initiator else self.rs
                if pub is None:
                    raise ValueError(f"pattern {pattern} needs the {'own' if who == initiator else 'remote'} static key")
                self._ss.mix_hash(pub)
        needs_s = any("s" in m for i, m in enumerate(self._messages) if (i % 2 == 0) == initiator)
        if needs_s and self.s is None:
            raise ValueError(f"pattern {pattern} sends this side's static key")
        self._step = 0
        self.complete = False

    def _dh(self, token: str) -> bytes:
        mine, theirs = token
        if not self.initiator:
            mine, theirs = theirs, mine
        priv = self.e if mine == "e" else self.s
        pub = self.re if theirs == "e" else self.rs
        if priv is None or pub is None:
            raise NoiseError(f"key for token {token} is missing")
        out = crypto.x25519(priv, pub)
        if out == b"\0" * 32:
            raise NoiseError("Diffie-Hellman produced the all-zero value")
        return out

    def _my_turn(self) -> bool:
        return (self._step % 2 == 0) == self.initiator

    def write_message(self, payload: bytes = b"") -> bytes:
        if self.complete or not self._my_turn():
            raise NoiseError("not this side's turn to write")
        out = b""
        for tok in self._messages[self._step]:
            if tok == "e":
                self.e = self.e or os.urandom(32)
                pub = crypto.x25519(self.e)
                out += pub
                self._ss.mix_hash(pub)
            elif tok == "s":
                out += self._ss.encrypt_and_hash(crypto.x25519(self.s))
            else:
                self._ss.mix_key(self._dh(tok))
        out += self._ss.encrypt_and_hash(payload)
        self._advance()
        return out

    def read_message(self, message: bytes) -> bytes:
        if self.complete or self._my_turn():
            raise NoiseError("not this side's turn to read")
        pos = 0
        for tok in self._messages[self._step]:
            if tok == "e":
                if len(message) < pos + 32:
                    raise NoiseError("message too short")
                self.re = message[pos:pos + 32]
                pos += 32
                self._ss.mix_hash(self.re)
            elif tok == "s":
                n = 48 if self._ss.cipher.has_key() else 32
                if len(message) < pos + n:
                    raise NoiseError("message too short")
                self.rs = self._ss.decrypt_and_hash(message[pos:pos + n])
                pos += n
            else:
                self._ss.mix_key(self._dh(tok))
        payload = self._ss.decrypt_and_hash(message[pos:])
        self._advance()
        return payload

    def _advance(self) -> None:
        self._step += 1
        self.complete = self._step == len(self._messages)

    @property
    def handshake_hash(self) -> bytes:
        return self._ss.h

    @property
    def chaining_key(self) -> bytes:
        return self._ss.ck

    def split(self) -> Tuple[CipherState, CipherState]:
        if not self.complete:
            raise NoiseError("handshake is not complete")
        return self._ss.split()


# ------------------------------------------------------------------------------------------------ tunnel on Noise IK
class ReplayWindow:
    """Sliding window over 64-bit packet counters (the scheme of RFC 6479): a counter is accepted once, counters
    older than ``size`` below the highest seen are refused."""

    def __init__(self, size: int = 2048):
        self.size, self.top, self.bits = size, -1, 0

    def check_and_update(self, n: int) -> bool:
        if n > self.top:
            shift = n - self.top
            self.bits = ((self.bits << shift) | 1) & ((1 << self.size) - 1) if shift < self.size else 1
            self.top = n
            return True
        off = self.top - n
        if off >= self.size or (self.bits >> off) & 1:
            return False
        self.bits |= 1 << off
        return True


class TunnelError(RuntimeError):
    pass


class TunnelPeer:
    """One end of a point-to-point tunnel in the shape of WireGuard: a one-round-trip Noise IK handshake between
    static X25519 keys, then data packets ``type(1) || counter(8, LE) || AEAD(payload)`` under directional keys, with a
    replay window on receive, rekey-required limits on message count and key age, empty keep-alive packets, and
    rx / tx byte counters. Packet types: 1 initiation, 2 response, 4 data."""

    REKEY_AFTER_MESSAGES, REJECT_AFTER_SECONDS = 2 ** 60, 180.0

    def __init__(self, static_private: bytes, peer_public: Optional[bytes] = None, clock: Callable[[], float] = time.time,
                 rekey_after_messages: Optional[int] = None):
        self.static, self.public, self.peer_public, self.clock = static_private, crypto.x25519(static_private), peer_public, clock
        self.rekey_after = rekey_after_messages or self.REKEY_AFTER_MESSAGES
        self._hs: Optional[NoiseHandshake] = None
        self._send = self._recv = None
        self._window = ReplayWindow()
        self._established = 0.0
        self.rx_bytes = self.tx_bytes = self.rx_packets = self.tx_packets = self.replays = 0

    # ---- handshake
    def initiate(self, ephemeral: Optional[bytes] = None) -> bytes:
        if self.peer_public is None:
            raise TunnelError("the initiator must know the peer's static key")
        self._hs = NoiseHandshake("IK", True, s=self.static, rs=self.peer_public, e=ephemeral, prologue=b"sneppx tunnel v1")
        stamp = struct.pack(">d", self.clock())
        return b"\x01" + self._hs.write_message(stamp)

    def respond(self, packet: bytes, ephemeral: Optional[bytes] = None, allowed_peers: Optional[Iterable[bytes]] = None) -> bytes:
        if packet[:1] != b"\x01":
            raise TunnelError("not an initiation packet")
        hs = NoiseHandshake("IK", False, s=self.static, e=ephemeral, prologue=b"sneppx tunnel v1")
        try:
            stamp = hs.read_message(packet[1:])
        except NoiseError as e:
            raise TunnelError(f"bad initiation: {e}") from e
        if allowed_peers is not None and hs.rs not in set(allowed_peers):
            raise TunnelError("unknown peer")
        if self.peer_public is not None and hs.rs != self.peer_public:
            raise TunnelError("unexpected peer key")
        if abs(struct.unpack(">d", stamp)[0] - self.clock()) > self.REJECT_AFTER_SECONDS:
            raise TunnelError("stale initiation")
        self.peer_public = hs.rs
        out = b"\x02" + hs.write_message(b"")
        i2r, r2i = hs.split()
        self._install(r2i, i2r)
        return out

    def finish(self, packet: bytes) -> None:
        if packet[:1] != b"\x02" or self._hs is None:
            raise TunnelError("not a response to a pending initiation")
        try:
            self._hs.read_message(packet[1:])
        except NoiseError as e:
            raise TunnelError(f"bad response: {e}") from e
        i2r, r2i = self._hs.split()
        self._hs = None
        self._install(i2r, r2i)

    def _install(self, send: CipherState, recv: CipherState) -> None:
        self._send, self._recv, self._window, self._established = send, recv, ReplayWindow(), self.clock()

    # ---- data
    @property
    def established(self) -> bool:
        return self._send is not None

    def needs_rekey(self) -> bool:
        return self.established and (self._send.n >= self.rekey_after or
                                     self.clock() - self._established >= self.REJECT_AFTER_SECONDS - 60.0)

    def send(self, payload: bytes) -> bytes:
        if not self.established:
            raise TunnelError("no session")
        if self._send.n >= self.rekey_after or self.clock() - self._established >= self.REJECT_AFTER_SECONDS:
            raise TunnelError("session keys are used up: handshake again")
        n = self._send.n
        pkt = b"\x04" + n.to_bytes(8, "little") + self._send.encrypt_with_ad(b"", payload)
        self.tx_bytes, self.tx_packets = self.tx_bytes + len(payload), self.tx_packets + 1
        return pkt

    def keepalive(self) -> bytes:
        return self.send(b"")

    def receive(self, packet: bytes) -> bytes:
        if not self.established:
            raise TunnelError("no session")
        if packet[:1] != b"\x04" or len(packet) < 9 + 16:
            raise TunnelError("not a data packet")
        if self.clock() - self._established >= self.REJECT_AFTER_SECONDS:
            raise TunnelError("session expired")
        n = int.from_bytes(packet[1:9], "little")
        try:
            payload = self._recv.decrypt_at(n, b"", packet[9:])
        except NoiseError as e:
            raise TunnelError("authentication failed") from e
        if not self._window.check_and_update(n):          # only authentic packets move the window
            self.replays += 1
            raise TunnelError("replayed or too old")
        self.rx_bytes, self.rx_packets = self.rx_bytes + len(payload), self.rx_packets + 1
        return payload

    def stats(self) -> dict:
        return {"rx_bytes": self.rx_bytes, "tx_bytes": self.tx_bytes, "rx_packets": self.rx_packets,
                "tx_packets": self.tx_packets, "replays": self.replays, "established": self.established}


# ------------------------------------------------------------------------------------------------ address lists
class IPBlocklist:
    """CIDR block list for IPv4 and IPv6 as two binary tries; ``check`` walks at most 32 / 128 bits."""

    def __init__(self, cidrs: Iterable[str] = ()):
        self._roots = {4: {}, 6: {}}
        self._nets: Dict[str, ipaddress._BaseNetwork] = {}
        for c in cidrs:
            self.add(c)

    @staticmethod
    def _bits(value: int, width: int, n: int):
        return ((value >> (width - 1 - i)) & 1 for i in range(n))

    def add(self, cidr: str) -> bool:
        net = ipaddress.ip_network(cidr, strict=False)
        if str(net) in self._nets:
            return False
        node = self._roots[net.version]
        for b in self._bits(int(net.network_address), net.max_prefixlen, net.prefixlen):
            node = node.setdefault(b, {})
        node["end"] = str(net)
        self._nets[str(net)] = net
        return True

    def remove(self, cidr: str) -> bool:
        net = ipaddress.ip_network(cidr, strict=False)
        if self._nets.pop(str(net), None) is None:
            return False
        path, node = [], self._roots[net.version]
        for b in self._bits(int(net.network_address), net.max_prefixlen, net.prefixlen):
            path.append((node, b))
            node = node[b]
        del node["end"]
        for parent, b in reversed(path):                  # prune branches that lead nowhere
            if parent[b]:
                break
            del parent[b]
        return True

    def match(self, ip) -> Optional[str]:
        """The shortest blocked prefix that covers ``ip`` (a string, an int for IPv4, or an ``ipaddress`` object)."""
        addr = ipaddress.ip_address(ip)
        node = self._roots[addr.version]
        if "end" in node:
            return node["end"]
        for b in self._bits(int(addr), addr.max_prefixlen, addr.max_prefixlen):
            node = node.get(b)
            if node is None:
                return None
            if "end" in node:
                return node["end"]
        return None

    def check(self, ip) -> bool:
        return self.match(ip) is not None

    def clear(self) -> None:
        self._roots, self._nets = {4: {}, 6: {}}, {}

    def __len__(self) -> int:
        return len(self._nets)

    def entries(self) -> List[str]:
        return sorted(self._nets)


# ------------------------------------------------------------------------------------------------ intrusion detection
@dataclass
class PacketInfo:
    src: str = ""
    dst: str = ""
    proto: str = ""            # tcp | udp | icmp | other
    sport: int = 0
    dport: int = 0
    flags: int = 0             # TCP flag byte
    payload: bytes = b""
    length: int = 0


def parse_ipv4_packet(packet: bytes) -> Optional[PacketInfo]:
    """Header fields of a raw IPv4 packet (TCP / UDP / ICMP); None for anything truncated or not version 4."""
    if len(packet) < 20 or packet[0] >> 4 != 4:
        return None
    ihl = (packet[0] & 0xF) * 4
    total = struct.unpack(">H", packet[2:4])[0]
    if ihl < 20 or len(packet) < ihl or total < ihl:
        return None
    body = packet[ihl:min(len(packet), total)]
    info = PacketInfo(str(ipaddress.IPv4Address(packet[12:16])), str(ipaddress.IPv4Address(packet[16:20])),
                      {6: "tcp", 17: "udp", 1: "icmp"}.get(packet[9], "other"), length=len(packet))
    if info.proto == "tcp":
        if len(body) < 20:
            return None
        info.sport, info.dport = struct.unpack(">HH", body[:4])
        off = (body[12] >> 4) * 4
        info.flags, info.payload = body[13], body[off:] if 20 <= off <= len(body) else b""
    elif info.proto == "udp":
        if len(body) < 8:
            return None
        info.sport, info.dport = struct.unpack(">HH", body[:4])
        info.payload = body[8:]
    else:
        info.payload = body[8:] if info.proto == "icmp" else body
    return info


@dataclass
class NidsRule:
    action: str
    proto: str
    dport: Optional[int]
    content: List[bytes]
    msg: str
    nocase: bool = False
    sid: int = 0


_RULE = re.compile(r"^\s*(alert|drop)\s+(tcp|udp|icmp|ip)\s+\S+\s+\S+\s+->\s+\S+\s+(\S+)\s*\((.*)\)\s*$")
TCP_FIN, TCP_SYN, TCP_RST, TCP_PSH, TCP_ACK, TCP_URG = 1, 2, 4, 8, 16, 32


def parse_nids_rule(line: str) -> NidsRule:
    """``alert tcp any any -> any 80 (msg:"..."; content:"..."; content:"|de ad|"; nocase; sid:1;)``: the subset of the
    Snort rule language with protocol, destination port, one or more contents (text or ``|hex|``), nocase, msg, sid."""
    m = _RULE.match(line)
    if not m:
        raise ValueError(f"bad rule: {line!r}")
    action, proto, dport, opts = m.groups()
    rule = NidsRule(action, proto, None if dport == "any" else int(dport), [], "")
    for opt in re.findall(r'(\w+)(?::\s*("(?:[^"\\]|\\.)*"|[^;]*))?\s*;', opts):
        k, v = opt[0], opt[1].strip()
        v = v[1:-1] if v.startswith('"') else v
        if k == "msg":
            rule.msg = v
        elif k == "content":
            out = b""
            for i, part in enumerate(v.split("|")):
                out += bytes.fromhex(part.replace(" ", "")) if i % 2 else part.encode()
            rule.content.append(out)
        elif k == "nocase":
            rule.nocase = True
        elif k == "sid":
            rule.sid = int(v)
    return rule


class Nids:
    """Signature and anomaly checks on raw IPv4 packets. Built-in detectors: blacklisted destination ports, TCP NULL /
    FIN-only / XMAS / SYN+FIN flag combinations, port scans (``scan_ports`` distinct destination ports from one
    source inside ``scan_window`` seconds), oversized ICMP echo payloads; plus content rules. ``analyze`` returns
    the alerts a packet raised; "drop" rules and built-in detectors mark the packet for dropping."""

    def __init__(self, scan_ports: int = 20, scan_window: float = 5.0, max_icmp_payload: int = 1024, max_alerts: int = 10000,
                 clock: Callable[[], float] = time.time):
        self.scan_ports, self.scan_window, self.max_icmp_payload, self.max_alerts, self.clock = \
            scan_ports, scan_window, max_icmp_payload, max_alerts, clock
        self.rules: List[NidsRule] = []
        self.port_blacklist: set = set()
        self.alerts: List[dict] = []
        self.packets = self.malformed = 0
        self._scan: Dict[str, Dict[int, float]] = {}

    def add_rule(self, line: str) -> NidsRule:
        r = parse_nids_rule(line)
        self.rules.append(r)
        return r

    def set_rules(self, path: str) -> int:
        """Replaces the rule list with the rules of a file (one per line, ``#`` comments); returns how many loaded."""
        with open(path) as f:
            lines = [l for l in (x.strip() for x in f) if l and not l.startswith("#")]
        self.rules = [parse_nids_rule(l) for l in lines]
        return len(self.rules)

    def add_port_blacklist(self, port: int) -> None:
        self.port_blacklist.add(int(port))

    def remove_port_blacklist(self, port: int) -> bool:
        if port in self.port_blacklist:
            self.port_blacklist.discard(port)
            return True
        return False

    def _alert(self, out: List[dict], kind: str, info: PacketInfo, msg: str, drop: bool, sid: int = 0) -> None:
        a = {"time": self.clock(), "kind": kind, "src": info.src, "dst": info.dst, "dport": info.dport, "msg": msg,
             "drop": drop, "sid": sid}
        out.append(a)
        if len(self.alerts) < self.max_alerts:
            self.alerts.append(a)

    def analyze(self, packet: bytes) -> List[dict]:
        self.packets += 1
        info = parse_ipv4_packet(packet)
        if info is None:
            self.malformed += 1
            return []
        out: List[dict] = []
        if info.proto in ("tcp", "udp") and info.dport in self.port_blacklist:
            self._alert(out, "port_blacklist", info, f"traffic to blacklisted port {info.dport}", True)
        if info.proto == "tcp":
            f = info.flags & 0x3F
            if f == 0:
                self._alert(out, "tcp_null_scan", info, "TCP segment with no flags", True)
            elif f == TCP_FIN:
                self._alert(out, "tcp_fin_scan", info, "TCP FIN without ACK", True)
            elif f == TCP_FIN | TCP_PSH | TCP_URG:
                self._alert(out, "tcp_xmas_scan", info, "TCP FIN+PSH+URG", True)
            elif f & TCP_SYN and f & TCP_FIN:
                self._alert(out, "tcp_syn_fin", info, "TCP SYN and FIN together", True)
            if f & TCP_SYN and not f & TCP_ACK:
                now = self.clock()
                seen = self._scan.setdefault(info.src, {})
                seen[info.dport] = now
                for p in [p for p, t in seen.items() if now - t > self.scan_window]:
                    del seen[p]
                if len(seen) >= self.scan_ports:
                    self._alert(out, "port_scan", info, f"{len(seen)} ports probed in {self.scan_window:g}s", True)
                    seen.clear()
        if info.proto == "icmp" and len(info.payload) > self.max_icmp_payload:
            self._alert(out, "icmp_oversize", info, f"ICMP payload of {len(info.payload)} bytes", True)
        for r in self.rules:
            if r.proto not in ("ip", info.proto) or (r.dport is not None and r.dport != info.dport):
                continue
            hay = info.payload.lower() if r.nocase else info.payload
            if all((c.lower() if r.nocase else c) in hay for c in r.content):
                self._alert(out, "rule", info, r.msg, r.action == "drop", r.sid)
        return out

    def should_drop(self, packet: bytes) -> bool:
        return any(a["drop"] for a in self.analyze(packet))

    def alert_count(self) -> int:
        return len(self.alerts)

    def last_alert_time(self) -> Optional[float]:
        return self.alerts[-1]["time"] if self.alerts else None

    def clear_alerts(self) -> None:
        self.alerts = []


# ------------------------------------------------------------------------------------------------ traffic shaping
def traffic_pad(data: bytes, block_size: int = 256) -> bytes:
    """Length-hiding padding: a 4-byte big-endian length, the data, then zeros up to a multiple of ``block_size``."""
    if block_size < 8:
        raise ValueError("block size must be at least 8")
    body = struct.pack(">I", len(data)) + data
    return body + b"\0" * (-len(body) % block_size)


def traffic_pad_to(data: bytes, target_size: int) -> bytes:
    if target_size < len(data) + 4:
        raise ValueError("target size is smaller than the framed data")
    return struct.pack(">I", len(data)) + data + b"\0" * (target_size - 4 - len(data))


def traffic_unpad(padded: bytes) -> bytes:
    if len(padded) < 4:
        raise ValueError("padded block is too short")
    n = struct.unpack(">I", padded[:4])[0]
    if n > len(padded) - 4 or any(padded[4 + n:]):
        raise ValueError("bad padding")
    return padded[4:4 + n]


def mtu_obfuscate(data: bytes, mtu: int = 1200, min_fragment: int = 64, rng: Optional[Callable[[int, int], int]] = None) -> List[bytes]:
    """Splits ``data`` into fragments of random sizes in [min_fragment, mtu - 6], each framed as index(2) || total(2) ||
    length(2) || bytes and padded to exactly ``mtu``, so every datagram on the wire has one size and the message
    length shows only as a fragment count. ``mtu_reassemble`` inverts it (any arrival order)."""
    import random
    pick = rng or random.SystemRandom().randint
    cap = mtu - 6
    if cap < min_fragment or min_fragment < 1:
        raise ValueError("mtu too small for the fragment header")
    pieces, pos = [], 0
    while pos < len(data) or not pieces:
        n = min(len(data) - pos, pick(min_fragment, cap))
        pieces.append(data[pos:pos + n])
        pos += n
    if len(pieces) > 0xFFFF:
        raise ValueError("message needs too many fragments")
    return [struct.pack(">HHH", i, len(pieces), len(p)) + p + os.urandom(cap - len(p)) for i, p in enumerate(pieces)]


def mtu_reassemble(fragments: Iterable[bytes]) -> bytes:
    parts: Dict[int, bytes] = {}
    total = None
    for f in fragments:
        i, t, n = struct.unpack(">HHH", f[:6])
        if n > len(f) - 6 or (total is not None and t != total):
            raise ValueError("inconsistent fragment")
        total, parts[i] = t, f[6:6 + n]
    if total is None or sorted(parts) != list(range(total)):
        raise ValueError("fragments missing")
    return b"".join(parts[i] for i in range(total))


# ------------------------------------------------------------------------------------------------ port knocking
def knock_sequence(secret: bytes, count: int = 4, epoch: Optional[int] = None, period_s: int = 30, low: int = 20000,
                   high: int = 60000, clock: Callable[[], float] = time.time) -> List[int]:
    """Time-based knock sequence both ends can compute: ports from HMAC-SHA256(secret, epoch || index), epoch = the
    current ``period_s`` interval."""
    epoch = int(clock() // period_s) if epoch is None else epoch
    out = []
    for i in range(count):
        d = crypto.hmac_sha256(secret, struct.pack(">QI", epoch, i))
        out.append(low + int.from_bytes(d[:4], "big") % (high - low))
    return out


def port_knock_verify(received: Sequence[int], expected: Sequence[int]) -> bool:
    """Exact, ordered match, compared without an early exit."""
    if len(received) != len(expected):
        return False
    diff = 0
    for a, b in zip(received, expected):
        diff |= a ^ b
    return diff == 0


class PortKnock:
    """Per-source knock tracker: a source that hits the expected ports in order, each within ``step_timeout`` seconds
    of the previous one, is opened for ``open_seconds``; a wrong port resets its progress."""

    def __init__(self, sequence: Sequence[int], step_timeout: float = 5.0, open_seconds: float = 30.0,
                 clock: Callable[[], float] = time.time):
        if not sequence:
            raise ValueError("empty knock sequence")
        self.sequence, self.step_timeout, self.open_seconds, self.clock = list(sequence), step_timeout, open_seconds, clock
        self._progress: Dict[str, Tuple[int, float]] = {}
        self._open: Dict[str, float] = {}

    def knock(self, source: str, port: int) -> bool:
        """Registers one knock; True when this knock completed the sequence."""
        now = self.clock()
        idx, last = self._progress.get(source, (0, now))
        if idx and now - last > self.step_timeout:
            idx = 0
        if port == self.sequence[idx]:
            idx += 1
        else:
            idx = 1 if port == self.sequence[0] else 0
        if idx == len(self.sequence):
            self._progress.pop(source, None)
            self._open[source] = now + self.open_seconds
            return True
        self._progress[source] = (idx, now)
        return False

    def is_open(self, source: str) -> bool:
        until = self._open.get(source)
        if until is None:
            return False
        if self.clock() >= until:
            del self._open[source]
            return False
        return True


# ------------------------------------------------------------------------------------------------ RPC authentication
class GrpcAuth:
    """Bearer-token call credentials for RPC metadata. ``renew`` swaps in a fresh random token and keeps the previous
    one valid for ``grace_s`` seconds so calls in flight still pass."""

    def __init__(self, token: Optional[bytes] = None, grace_s: float = 30.0, clock: Callable[[], float] = time.time):
        self.grace_s, self.clock = grace_s, clock
        self._token: Optional[bytes] = None
        self._previous: Optional[Tuple[bytes, float]] = None
        self.generation = 0
        if token is not None:
            self.set_token(token)

    def has_token(self) -> bool:
        return self._token is not None

    def set_token(self, token: bytes) -> None:
        if not token:
            raise ValueError("empty token")
        self._token, self._previous = bytes(token), None
        self.generation += 1

    def get_token(self) -> Optional[bytes]:
        return self._token

    def renew(self, nbytes: int = 32) -> bytes:
        if self._token is not None:
            self._previous = (self._token, self.clock() + self.grace_s)
        self._token = base64.urlsafe_b64encode(os.urandom(nbytes)).rstrip(b"=")
        self.generation += 1
        return self._token

    def verify(self, received: bytes) -> bool:
        if self._token is None or not received:
            return False
        ok = _hmac.compare_digest(crypto.sha256(received), crypto.sha256(self._token))
        if self._previous is not None:
            if self.clock() < self._previous[1]:
                ok |= _hmac.compare_digest(crypto.sha256(received), crypto.sha256(self._previous[0]))
            else:
                self._previous = None
        return ok

    def client_metadata(self) -> List[Tuple[str, str]]:
        if self._token is None:
            raise RuntimeError("no token set")
        return [("authorization", "Bearer " + self._token.decode())]

    def verify_metadata(self, metadata: Iterable[Tuple[str, str]]) -> bool:
        for k, v in metadata:
            if k.lower() == "authorization" and v.lower().startswith("bearer "):
                return self.verify(v[7:].strip().encode())
        return False


# ------------------------------------------------------------------------------------------------ DNS over HTTPS
DNS_A, DNS_CNAME, DNS_AAAA = 1, 5, 28


def dns_build_query(hostname: str, qtype: int = DNS_A, query_id: int = 0) -> bytes:
    """RFC 1035 query message (recursion desired). RFC 8484 asks for id 0 so that HTTP caches can share answers."""
    name = b""
    for label in hostname.rstrip(".").split("."):
        raw = label.encode("idna")
        if not 0 < len(raw) < 64:
            raise ValueError(f"bad label in {hostname!r}")
        name += bytes([len(raw)]) + raw
    return struct.pack(">HHHHHH", query_id, 0x0100, 1, 0, 0, 0) + name + b"\0" + struct.pack(">HH", qtype, 1)


def _dns_name(msg: bytes, pos: int, depth: int = 0) -> Tuple[str, int]:
    labels, jumped_end = [], None
    while True:
        if pos >= len(msg) or depth > 16:
            raise ValueError("bad DNS name")
        n = msg[pos]
        if n == 0:
            pos += 1
            break
        if n & 0xC0 == 0xC0:                                # compression pointer
            if pos + 1 >= len(msg):
                raise ValueError("bad DNS name")
            ptr = ((n & 0x3F) << 8) | msg[pos + 1]
            if jumped_end is None:
                jumped_end = pos + 2
            pos, depth = ptr, depth + 1
            continue
        labels.append(msg[pos + 1:pos + 1 + n].decode("ascii", "replace"))
        pos += 1 + n
    return ".".join(labels), (jumped_end if jumped_end is not None else pos)


def dns_parse_response(msg: bytes) -> dict:
    """{"id", "rcode", "answers": [{"name", "type", "ttl", "data"}]} with A / AAAA addresses and CNAME targets decoded."""
    if len(msg) < 12:
        raise ValueError("truncated DNS message")
    qid, flags, qd, an, _, _ = struct.unpack(">HHHHHH", msg[:12])
    if not flags & 0x8000:
        raise ValueError("not a response")
    pos = 12
    for _ in range(qd):
        _, pos = _dns_name(msg, pos)
        pos += 4
    answers = []
    for _ in range(an):
        name, pos = _dns_name(msg, pos)
        if pos + 10 > len(msg):
            raise ValueError("truncated DNS record")
        rtype, _, ttl, rdlen = struct.unpack(">HHIH", msg[pos:pos + 10])
        pos += 10
        rdata = msg[pos:pos + rdlen]
        if len(rdata) != rdlen:
            raise ValueError("truncated DNS record")
        if rtype == DNS_A and rdlen == 4:
            data = str(ipaddress.IPv4Address(rdata))
        elif rtype == DNS_AAAA and rdlen == 16:
            data = str(ipaddress.IPv6Address(rdata))
        elif rtype == DNS_CNAME:
            data = _dns_name(msg, pos)[0]
        else:
            data = rdata
        answers.append({"name": name, "type": rtype, "ttl": ttl, "data": data})
        pos += rdlen
    return {"id": qid, "rcode": flags & 0xF, "answers": answers}


def _https_transport(url: str, body: Optional[bytes]) -> bytes:
    import urllib.request
    req = urllib.request.Request(url, data=body, headers={"Accept": "application/dns-message",
                                                          **({"Content-Type": "application/dns-message"} if body else {})})
    with urllib.request.urlopen(req, timeout=5.0) as r:
        return r.read()


class DohResolver:
    """RFC 8484 client: GET ``?dns=<base64url query>`` (or POST of the wire message) against ``resolver_url``; answers
    are cached until their smallest TTL runs out. ``transport(url, body) -> bytes`` performs the HTTPS exchange."""

    def __init__(self, resolver_url: str = "https://dns.example/dns-query", use_post: bool = False,
                 transport: Callable[[str, Optional[bytes]], bytes] = _https_transport, clock: Callable[[], float] = time.time):
        self.set_resolver(resolver_url)
        self.use_post, self.transport, self.clock = use_post, transport, clock
        self._cache: Dict[Tuple[str, int], Tuple[float, List[str]]] = {}
        self.queries = self.cache_hits = 0

    def set_resolver(self, url: str) -> None:
        if not url.lower().startswith("https://"):
            raise ValueError("a DoH resolver must be an https:// URL")
        self.resolver_url = url

    def resolve(self, hostname: str, qtype: int = DNS_A) -> List[str]:
        key = (hostname.lower().rstrip("."), qtype)
        hit = self._cache.get(key)
        if hit and self.clock() < hit[0]:
            self.cache_hits += 1
            return list(hit[1])
        q = dns_build_query(hostname, qtype)
        if self.use_post:
            raw = self.transport(self.resolver_url, q)
        else:
            raw = self.transport(self.resolver_url + "?dns=" + base64.urlsafe_b64encode(q).rstrip(b"=").decode(), None)
        self.queries += 1
        resp = dns_parse_response(raw)
        if resp["rcode"] != 0:
            return []
        recs = [a for a in resp["answers"] if a["type"] == qtype]
        addrs = [a["data"] for a in recs]
        if addrs:
            self._cache[key] = (self.clock() + min(a["ttl"] for a in resp["answers"]), addrs)
        return addrs

    def resolve_batch(self, hostnames: Sequence[str], qtype: int = DNS_A) -> Dict[str, List[str]]:
        return {h: self.resolve(h, qtype) for h in hostnames}


# ------------------------------------------------------------------------------------------------ certificate transparency
def ct_leaf_hash(leaf: bytes) -> bytes:
    return hashlib.sha256(b"\x00" + leaf).digest()


def _ct_node(left: bytes, right: bytes) -> bytes:
    return hashlib.sha256(b"\x01" + left + right).digest()


def _split_point(n: int) -> int:
    k = 1
    while k * 2 < n:
        k *= 2
    return k


def ct_merkle_root(leaves: Sequence[bytes]) -> bytes:
    """RFC 6962 section 2.1 Merkle tree hash of the leaf inputs."""
    if not leaves:
        return hashlib.sha256(b"").digest()
    if len(leaves) == 1:
        return ct_leaf_hash(leaves[0])
    k = _split_point(len(leaves))
    return _ct_node(ct_merkle_root(leaves[:k]), ct_merkle_root(leaves[k:]))


def ct_inclusion_proof(leaves: Sequence[bytes], index: int) -> List[bytes]:
    """Audit path of leaf ``index`` (RFC 6962 section 2.1.1), lowest node first."""
    n = len(leaves)
    if not 0 <= index < n:
        raise IndexError(index)
    if n == 1:
        return []
    k = _split_point(n)
    if index < k:
        return ct_inclusion_proof(leaves[:k], index) + [ct_merkle_root(leaves[k:])]
    return ct_inclusion_proof(leaves[k:], index - k) + [ct_merkle_root(leaves[:k])]


def ct_verify_inclusion(leaf: bytes, index: int, tree_size: int, proof: Sequence[bytes], root: bytes) -> bool:
    """Recomputes the root from a leaf and its audit path (the algorithm of RFC 9162 section 2.1.3.2)."""
    if not 0 <= index < tree_size:
        return False
    fn, sn, r = index, tree_size - 1, ct_leaf_hash(leaf)
    for p in proof:
        if sn == 0:
            return False
        if fn & 1 or fn == sn:
            r = _ct_node(p, r)
            if not fn & 1:
                while fn and not fn & 1:
                    fn, sn = fn >> 1, sn >> 1
        else:
            r = _ct_node(r, p)
        fn, sn = fn >> 1, sn >> 1
    return sn == 0 and _hmac.compare_digest(r, root)


def ct_consistency_proof(leaves: Sequence[bytes], first: int) -> List[bytes]:
    """Proof that the tree over ``leaves[:first]`` is a prefix of the tree over all ``leaves`` (RFC 6962 section 2.1.2)."""
    n = len(leaves)
    if not 0 < first <= n:
        raise ValueError("first tree size out of range")

    def sub(m: int, d: Sequence[bytes], whole: bool) -> List[bytes]:
        if m == len(d):
            return [] if whole else [ct_merkle_root(d)]
        k = _split_point(len(d))
        if m <= k:
            return sub(m, d[:k], whole) + [ct_merkle_root(d[k:])]
        return sub(m - k, d[k:], False) + [ct_merkle_root(d[:k])]

    return sub(first, leaves, True)


def ct_verify_consistency(first: int, second: int, first_root: bytes, second_root: bytes, proof: Sequence[bytes]) -> bool:
    """RFC 9162 section 2.1.4.2."""
    if first == second:
        return not proof and first_root == second_root
    if not 0 < first < second:
        return False
    path = list(proof)
    if first & (first - 1) == 0:
        path = [first_root] + path
    if not path:
        return False
    fn, sn = first - 1, second - 1
    while fn & 1:
        fn, sn = fn >> 1, sn >> 1
    fr = sr = path[0]
    for c in path[1:]:
        if sn == 0:
            return False
        if fn & 1 or fn == sn:
            fr, sr = _ct_node(c, fr), _ct_node(c, sr)
            if not fn & 1:
                while fn and not fn & 1:
                    fn, sn = fn >> 1, sn >> 1
        else:
            sr = _ct_node(sr, c)
        fn, sn = fn >> 1, sn >> 1
    return sn == 0 and _hmac.compare_digest(fr, first_root) and _hmac.compare_digest(sr, second_root)


@dataclass
class SignedCertificateTimestamp:
    """The v1 SCT structure of RFC 6962 section 3.2: version(1) log_id(32) timestamp(8, ms) extensions(2+n)
    hash_alg(1) sig_alg(1) signature(2+n)."""

    log_id: bytes
    timestamp_ms: int
    extensions: bytes = b""
    hash_alg: int = 4           # sha256
    sig_alg: int = 7            # ed25519 in the TLS SignatureAlgorithm registry
    signature: bytes = b""
    version: int = 0

    def encode(self) -> bytes:
        return (bytes([self.version]) + self.log_id + struct.pack(">Q", self.timestamp_ms) +
                struct.pack(">H", len(self.extensions)) + self.extensions + bytes([self.hash_alg, self.sig_alg]) +
                struct.pack(">H", len(self.signature)) + self.signature)

    @classmethod
    def parse(cls, raw: bytes) -> "SignedCertificateTimestamp":
        if len(raw) < 47:
            raise ValueError("SCT too short")
        version, log_id, ts = raw[0], raw[1:33], struct.unpack(">Q", raw[33:41])[0]
        n = struct.unpack(">H", raw[41:43])[0]
        ext, pos = raw[43:43 + n], 43 + n
        if pos + 4 > len(raw):
            raise ValueError("SCT truncated")
        h, s, m = raw[pos], raw[pos + 1], struct.unpack(">H", raw[pos + 2:pos + 4])[0]
        sig = raw[pos + 4:pos + 4 + m]
        if len(ext) != n or len(sig) != m or pos + 4 + m != len(raw):
            raise ValueError("SCT length fields do not add up")
        return cls(log_id, ts, ext, h, s, sig, version)

    def signed_data(self, cert_der: bytes) -> bytes:
        """The digitally-signed struct for an X.509 entry: version, signature_type 0, timestamp, entry_type 0,
        24-bit length + certificate, extensions."""
        return (bytes([self.version, 0]) + struct.pack(">Q", self.timestamp_ms) + b"\0\0" + len(cert_der).to_bytes(3, "big") +
                cert_der + struct.pack(">H", len(self.extensions)) + self.extensions)


def ct_issue_sct(cert_der: bytes, log_seed: bytes, timestamp_ms: int, extensions: bytes = b"") -> SignedCertificateTimestamp:
    """What a log with the Ed25519 key ``log_seed`` returns for a submitted certificate (log id = SHA-256 of its key)."""
    pub = crypto.ed25519_public_key(log_seed)
    sct = SignedCertificateTimestamp(hashlib.sha256(pub).digest(), timestamp_ms, extensions)
    sct.signature = crypto.ed25519_sign(log_seed, sct.signed_data(cert_der))
    return sct


def ct_verify_sct(sct, cert_der: bytes, log_keys: Dict[bytes, bytes], now_ms: Optional[int] = None) -> bool:
    """True when the SCT (object or bytes) is a v1 SCT from a known log (``log_keys``: log id -> Ed25519 public key),
    is not dated in the future and its signature covers this certificate. Logs that sign with ECDSA P-256 cannot be
    checked here: this package has no P-256 arithmetic."""
    try:
        s = sct if isinstance(sct, SignedCertificateTimestamp) else SignedCertificateTimestamp.parse(sct)
    except ValueError:
        return False
    key = log_keys.get(s.log_id)
    if key is None or s.version != 0 or s.sig_alg != 7 or len(s.signature) != 64:
        return False
    if now_ms is not None and s.timestamp_ms > now_ms:
        return False
    return crypto.ed25519_verify(key, s.signed_data(cert_der), s.signature)


def ct_verify_all_scts(scts: Iterable, cert_der: bytes, log_keys: Dict[bytes, bytes], now_ms: Optional[int] = None,
                       required: int = 2) -> Tuple[bool, List[bool]]:
    """(policy met, result per SCT): the policy asks for ``required`` valid SCTs from distinct logs."""
    results, logs = [], set()
    for raw in scts:
        ok = ct_verify_sct(raw, cert_der, log_keys, now_ms)
        results.append(ok)
        if ok:
            s = raw if isinstance(raw, SignedCertificateTimestamp) else SignedCertificateTimestamp.parse(raw)
            logs.add(s.log_id)
    return len(logs) >= required, results
