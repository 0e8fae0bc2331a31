"""QUIC version 1 packet protection (RFC 9001) and packet-number coding (RFC 9000 section 17.1, appendix A).

The pieces another QUIC stack has to agree with bit for bit:

* Initial secrets from the client's destination connection id (HKDF-Extract with the version 1 salt, then
  HKDF-Expand-Label "client in" / "server in"), and from any traffic secret the key, IV and header-protection key
  ("quic key", "quic iv", "quic hp") and the next-generation secret of a key update ("quic ku").
* AEAD protection of the payload with nonce = IV xor packet number and the unprotected header as associated data:
  AES-128-GCM (the suite of Initial packets) and ChaCha20-Poly1305.
* Header protection: a 16-byte sample of the ciphertext, taken 4 bytes after the start of the packet-number field,
  gives a 5-byte mask (AES-ECB of the sample, or ChaCha20 keyed by the sample's counter and nonce) that hides the low
  bits of the first byte and the packet-number bytes.
* The Retry integrity tag (AES-128-GCM over the pseudo-packet with the fixed version 1 key and nonce).
* Truncated packet numbers: the shortest encoding that the peer can expand given the largest acknowledged number, and
  the expansion around the largest number received.

AES-128 and GHASH are written here in Python, since the native library carries AES-256-GCM only and these run per
handshake packet, not per tensor; ChaCha20-Poly1305, ChaCha20 and HKDF come from ``security.crypto``. The UDP transport
in ``utils/quic.py`` keeps its own simpler framing; this module is the wire-exact layer for talking to, or inspecting
traffic of, other QUIC implementations. The reference has no counterpart beyond the empty shell in
net/quic/quic_transport.c:30-119.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Optional, Tuple

from ..security import crypto
from ..security.network_ext import hkdf_expand_label, hkdf_extract

INITIAL_SALT_V1 = bytes.fromhex("38762cf7f55934b34d179ae6a4c80cadccbb7f0a")
RETRY_KEY_V1 = bytes.fromhex("be0c690b9f66575a1d766b54e368c84e")
RETRY_NONCE_V1 = bytes.fromhex("461599d35d632bf2239825bb")
AES_128_GCM, CHACHA20_POLY1305 = "aes-128-gcm", "chacha20-poly1305"
TAG_LEN = 16


class ProtectionError(ValueError):
    """A packet that fails authentication or is too short to carry a header-protection sample."""


# ------------------------------------------------------------------------------------------------------- AES-128
def _xtime(a: int) -> int:
    a <<= 1
    return (a ^ 0x11B) & 0xFF if a & 0x100 else a


def _make_sbox():
    # multiplicative inverse in GF(2^8) through the generator 3, then the affine map of FIPS 197 section 5.1.1
    exp, log = [0] * 255, [0] * 256
    x = 1
    for i in range(255):
        exp[i], log[x] = x, i
        x ^= _xtime(x)
    box = [0] * 256
    for v in range(256):
        inv = 0 if v == 0 else exp[(255 - log[v]) % 255]
        r = inv
        for s in range(1, 5):
            r ^= ((inv << s) | (inv >> (8 - s))) & 0xFF
        box[v] = r ^ 0x63
    return bytes(box)


_SBOX = _make_sbox()
_MUL2 = bytes(_xtime(i) for i in range(256))
_MUL3 = bytes(_xtime(i) ^ i for i in range(256))


class Aes128:
    """The AES-128 forward cipher (FIPS 197); GCM and header protection need encryption only."""

    def __init__(self, key: bytes):
        if len(key) != 16:
            raise ValueError("AES-128 takes a 16-byte key")
        w = [key[4 * i:4 * i + 4] for i in range(4)]
        rcon = 1
        for i in range(4, 44):
            t = w[i - 1]
            if i % 4 == 0:
                t = bytes((_SBOX[t[1]] ^ rcon, _SBOX[t[2]], _SBOX[t[3]], _SBOX[t[0]]))
                rcon = _xtime(rcon)
            w.append(bytes(a ^ b for a, b in zip(w[i - 4], t)))
        self._rk = [b"".join(w[4 * r:4 * r + 4]) for r in range(11)]

    def encrypt_block(self, block: bytes) -> bytes:
        if len(block) != 16:
            raise ValueError("AES works on 16-byte blocks")
        s = bytes(a ^ b for a, b in zip(block, self._rk[0]))
        for rnd in range(1, 11):
            s = bytes(_SBOX[s[(c * 4 + r + 4 * r) % 16]] for c in range(4) for r in range(4))   # SubBytes + ShiftRows
            if rnd < 10:
                out = bytearray(16)
                for c in range(4):
                    a0, a1, a2, a3 = s[4 * c:4 * c + 4]
                    out[4 * c] = _MUL2[a0] ^ _MUL3[a1] ^ a2 ^ a3
                    out[4 * c + 1] = a0 ^ _MUL2[a1] ^ _MUL3[a2] ^ a3
                    out[4 * c + 2] = a0 ^ a1 ^ _MUL2[a2] ^ _MUL3[a3]
                    out[4 * c + 3] = _MUL3[a0] ^ a1 ^ a2 ^ _MUL2[a3]
                s = bytes(out)
            s = bytes(a ^ b for a, b in zip(s, self._rk[rnd]))
        return s


# ----------------------------------------------------------------------------------------------------------- GCM
_R = 0xE1 << 120


def _gf_mul(x: int, y: int) -> int:
    """Product in GF(2^128) with GCM's bit order (NIST SP 800-38D section 6.3)."""
    z = 0
    for i in range(127, -1, -1):
        if (x >> i) & 1:
            z ^= y
        y = (y >> 1) ^ _R if y & 1 else y >> 1
    return z


def _ghash(h: int, aad: bytes, ct: bytes) -> int:
    y = 0
    for data in (aad, ct):
        for i in range(0, len(data), 16):
            y = _gf_mul(y ^ int.from_bytes(data[i:i + 16].ljust(16, b"\0"), "big"), h)
    return _gf_mul(y ^ ((len(aad) * 8) << 64 | (len(ct) * 8)), h)


def _gcm_ctr(aes: Aes128, iv: bytes, data: bytes) -> bytes:
    out = bytearray()
    for i in range(0, len(data), 16):
        ks = aes.encrypt_block(iv + struct.pack(">I", 2 + i // 16))
        out += bytes(a ^ b for a, b in zip(data[i:i + 16], ks))
    return bytes(out)


def aes128_gcm_encrypt(key: bytes, iv: bytes, plaintext: bytes, aad: bytes = b"") -> bytes:
    """Ciphertext followed by the 16-byte tag; ``iv`` is the 12-byte nonce."""
    if len(iv) != 12:
        raise ValueError("GCM here takes a 12-byte nonce")
    aes = Aes128(key)
    h = int.from_bytes(aes.encrypt_block(b"\0" * 16), "big")
    ct = _gcm_ctr(aes, iv, plaintext)
    tag = _ghash(h, aad, ct) ^ int.from_bytes(aes.encrypt_block(iv + b"\0\0\0\1"), "big")
    return ct + tag.to_bytes(16, "big")


def aes128_gcm_decrypt(key: bytes, iv: bytes, sealed: bytes, aad: bytes = b"") -> bytes:
    if len(iv) != 12 or len(sealed) < TAG_LEN:
        raise ProtectionError("sealed data shorter than a tag")
    aes = Aes128(key)
    h = int.from_bytes(aes.encrypt_block(b"\0" * 16), "big")
    ct, tag = sealed[:-TAG_LEN], sealed[-TAG_LEN:]
    want = _ghash(h, aad, ct) ^ int.from_bytes(aes.encrypt_block(iv + b"\0\0\0\1"), "big")
    if not crypto.ct_equal(want.to_bytes(16, "big"), tag):
        raise ProtectionError("authentication failed")
    return _gcm_ctr(aes, iv, ct)


# ------------------------------------------------------------------------------------------------ key derivation
@dataclass(frozen=True)
class PacketKeys:
    """What protects one direction of one encryption level."""
    suite: str
    key: bytes
    iv: bytes
    hp: bytes
    secret: bytes

    def next_generation(self) -> "PacketKeys":
        """Keys after a key update (RFC 9001 section 6.1): a new secret, key and IV; the header key stays."""
        nxt = hkdf_expand_label(self.secret, "quic ku", b"", len(self.secret))
        k = derive_packet_keys(nxt, self.suite)
        return PacketKeys(self.suite, k.key, k.iv, self.hp, nxt)


def derive_packet_keys(secret: bytes, suite: str = AES_128_GCM) -> PacketKeys:
    klen = {AES_128_GCM: 16, CHACHA20_POLY1305: 32}[suite]
    return PacketKeys(suite, hkdf_expand_label(secret, "quic key", b"", klen), hkdf_expand_label(secret, "quic iv", b"", 12),
                      hkdf_expand_label(secret, "quic hp", b"", klen), secret)


def initial_secrets(client_dcid: bytes, salt: bytes = INITIAL_SALT_V1) -> Tuple[bytes, bytes]:
    """(client_initial_secret, server_initial_secret) for the connection id of the client's first Initial packet."""
    initial = hkdf_extract(salt, client_dcid)
    return hkdf_expand_label(initial, "client in", b"", 32), hkdf_expand_label(initial, "server in", b"", 32)


def initial_keys(client_dcid: bytes, is_client: bool) -> Tuple[PacketKeys, PacketKeys]:
    """(send keys, receive keys) of the Initial level for one endpoint."""
    c, s = (derive_packet_keys(x) for x in initial_secrets(client_dcid))
    return (c, s) if is_client else (s, c)


# ---------------------------------------------------------------------------------------------- packet numbers
def encode_packet_number(full_pn: int, largest_acked: Optional[int] = None) -> bytes:
    """The shortest field (1 - 4 bytes) that covers twice the range of packets in flight (RFC 9000 appendix A.2)."""
    unacked = full_pn + 1 if largest_acked is None else full_pn - largest_acked
    if unacked <= 0:
        raise ValueError("a packet number at or below the largest acknowledged one is never sent")
    need = max(1, ((2 * unacked).bit_length() + 7) // 8)        # bits to express twice the range, in whole bytes
    if need > 4:
        raise ValueError("more than 2^31 packets in flight")
    return (full_pn & ((1 << (8 * need)) - 1)).to_bytes(need, "big")


def decode_packet_number(largest_pn: int, truncated: int, pn_nbits: int) -> int:
    """The full number closest to one past the largest received (RFC 9000 appendix A.3)."""
    expected = largest_pn + 1
    win = 1 << pn_nbits
    hwin, mask = win // 2, win - 1
    candidate = (expected & ~mask) | truncated
    if candidate <= expected - hwin and candidate < (1 << 62) - win:
        return candidate + win
    if candidate > expected + hwin and candidate >= win:
        return candidate - win
    return candidate


# ---------------------------------------------------------------------------------------------------- protection
def _hp_mask(keys: PacketKeys, sample: bytes) -> bytes:
    if keys.suite == AES_128_GCM:
        return Aes128(keys.hp).encrypt_block(sample)[:5]
    counter = struct.unpack("<I", sample[:4])[0]
    return crypto.chacha20(keys.hp, sample[4:16], b"\0" * 5, counter)


def _aead(keys: PacketKeys, pn: int, data: bytes, aad: bytes, seal: bool) -> bytes:
    nonce = (int.from_bytes(keys.iv, "big") ^ pn).to_bytes(12, "big")
    if keys.suite == AES_128_GCM:
        return (aes128_gcm_encrypt if seal else aes128_gcm_decrypt)(keys.key, nonce, data, aad)
    if seal:
        return crypto.aead_encrypt(keys.key, nonce, data, aad)
    try:
        return crypto.aead_decrypt(keys.key, nonce, data, aad)
    except Exception as e:
        raise ProtectionError("authentication failed") from e


def protect_packet(keys: PacketKeys, header: bytes, pn_length: int, full_pn: int, payload: bytes) -> bytes:
    """``header`` is the complete unprotected header ending in the ``pn_length``-byte packet number (its low two bits of
    the first byte already say ``pn_length - 1``; a long header's Length field already counts packet number, payload
    and tag). Returns the protected packet."""
    if not 1 <= pn_length <= 4 or (header[0] & 0x03) != pn_length - 1:
        raise ValueError("first byte and packet-number length disagree")
    if len(payload) + pn_length < 4:
        raise ValueError("payload too short for a header-protection sample: pad it (RFC 9001 section 5.4.2)")
    sealed = _aead(keys, full_pn, payload, header, True)
    pn_off = len(header) - pn_length
    sample = sealed[4 - pn_length:4 - pn_length + 16]
    mask = _hp_mask(keys, sample)
    out = bytearray(header)
    out[0] ^= mask[0] & (0x0F if header[0] & 0x80 else 0x1F)
    for i in range(pn_length):
        out[pn_off + i] ^= mask[1 + i]
    return bytes(out) + sealed


def unprotect_packet(keys: PacketKeys, packet: bytes, pn_offset: int, largest_pn: int = -1) -> Tuple[bytes, int, bytes]:
    """Remove header protection, expand the packet number around ``largest_pn`` and open the payload.
    ``pn_offset`` is where the packet-number field starts (after the Length field of a long header, after the
    destination connection id of a short one); ``packet`` ends where this QUIC packet ends. Returns
    (unprotected header, full packet number, payload)."""
    if len(packet) < pn_offset + 4 + 16:
        raise ProtectionError("packet too short to sample")
    mask = _hp_mask(keys, packet[pn_offset + 4:pn_offset + 20])
    hdr = bytearray(packet[:pn_offset + 4])
    hdr[0] ^= mask[0] & (0x0F if hdr[0] & 0x80 else 0x1F)
    pn_length = (hdr[0] & 0x03) + 1
    for i in range(pn_length):
        hdr[pn_offset + i] ^= mask[1 + i]
    header = bytes(hdr[:pn_offset + pn_length])
    truncated = int.from_bytes(header[pn_offset:], "big")
    full_pn = decode_packet_number(largest_pn, truncated, 8 * pn_length)
    return header, full_pn, _aead(keys, full_pn, packet[pn_offset + pn_length:], header, False)


# --------------------------------------------------------------------------------------------------------- Retry
def retry_integrity_tag(original_dcid: bytes, retry_without_tag: bytes) -> bytes:
    """RFC 9001 section 5.8: the tag is AES-128-GCM over nothing, with the pseudo-packet as associated data."""
    pseudo = bytes([len(original_dcid)]) + original_dcid + retry_without_tag
    return aes128_gcm_encrypt(RETRY_KEY_V1, RETRY_NONCE_V1, b"", pseudo)


def verify_retry(original_dcid: bytes, retry_packet: bytes) -> bool:
    if len(retry_packet) < TAG_LEN + 7:
        return False
    return crypto.ct_equal(retry_integrity_tag(original_dcid, retry_packet[:-TAG_LEN]), retry_packet[-TAG_LEN:])


# ------------------------------------------------------------------------------------------------ header helpers
def _varint(v: int) -> bytes:
    for bits, prefix in ((6, 0), (14, 1), (30, 2), (62, 3)):
        if v < (1 << bits):
            n = 1 << prefix
            return ((prefix << (8 * n - 2)) | v).to_bytes(n, "big")
    raise ValueError("varint out of range")


def _read_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    n = 1 << (buf[pos] >> 6)
    return int.from_bytes(buf[pos:pos + n], "big") & ((1 << (8 * n - 2)) - 1), pos + n


LONG_INITIAL, LONG_0RTT, LONG_HANDSHAKE, LONG_RETRY = 0, 1, 2, 3


def build_long_header(packet_type: int, dcid: bytes, scid: bytes, pn: bytes, payload_len: int, token: bytes = b"",
                      version: int = 1) -> bytes:
    """An unprotected long header for Initial / 0-RTT / Handshake packets. ``payload_len`` is the plaintext length of the
    frames; the Length field written is packet number + payload + tag, always as a 2-byte varint so that the header's
    size does not depend on it."""
    first = 0xC0 | (packet_type << 4) | (len(pn) - 1)
    out = bytes([first]) + struct.pack(">I", version) + bytes([len(dcid)]) + dcid + bytes([len(scid)]) + scid
    if packet_type == LONG_INITIAL:
        out += _varint(len(token)) + token
    length = len(pn) + payload_len + TAG_LEN
    if length >= 1 << 14:
        raise ValueError("packet longer than a 2-byte Length field")
    return out + (0x4000 | length).to_bytes(2, "big") + pn


def parse_long_header(packet: bytes) -> dict:
    """The unprotected part of a long header: type, version, connection ids, token, and where the packet-number field
    and the end of this packet are (several packets may share a datagram)."""
    if not packet or not packet[0] & 0x80:
        raise ValueError("not a long header")
    try:
        return _parse_long_header(packet)
    except (IndexError, struct.error):
        raise ValueError("truncated long header") from None


def _parse_long_header(packet: bytes) -> dict:
    ptype = (packet[0] >> 4) & 3
    version = struct.unpack(">I", packet[1:5])[0]
    pos = 5
    dcid = packet[pos + 1:pos + 1 + packet[pos]]
    pos += 1 + len(dcid)
    scid = packet[pos + 1:pos + 1 + packet[pos]]
    pos += 1 + len(scid)
    token = b""
    if ptype == LONG_RETRY:
        return {"type": ptype, "version": version, "dcid": dcid, "scid": scid, "token": packet[pos:-TAG_LEN],
                "pn_offset": None, "end": len(packet)}
    if ptype == LONG_INITIAL:
        tlen, pos = _read_varint(packet, pos)
        token = packet[pos:pos + tlen]
        pos += tlen
    length, pos = _read_varint(packet, pos)
    return {"type": ptype, "version": version, "dcid": dcid, "scid": scid, "token": token, "pn_offset": pos,
            "end": pos + length}


def build_short_header(dcid: bytes, pn: bytes, key_phase: int = 0, spin: int = 0) -> bytes:
    return bytes([0x40 | (spin << 5) | (key_phase << 2) | (len(pn) - 1)]) + dcid + pn


class PacketProtector:
    """One endpoint's view of one encryption level: seals outgoing packets with the shortest packet number that the
    peer can expand, opens incoming ones, tracks the largest number received, and follows the peer through key updates
    (a packet whose key-phase bit differs is tried with the next generation of receive keys; on success both directions
    move on, RFC 9001 section 6)."""

    def __init__(self, send: PacketKeys, recv: PacketKeys):
        self.send, self.recv = send, recv
        self.next_pn, self.largest_acked, self.largest_received = 0, None, -1
        self.key_phase = 0

    def on_ack(self, largest_acked: int) -> None:
        if self.largest_acked is None or largest_acked > self.largest_acked:
            self.largest_acked = largest_acked

    def seal_long(self, packet_type: int, dcid: bytes, scid: bytes, payload: bytes, token: bytes = b"") -> bytes:
        pn = encode_packet_number(self.next_pn, self.largest_acked)
        payload = payload.ljust(max(len(payload), 4 - len(pn)), b"\0")
        hdr = build_long_header(packet_type, dcid, scid, pn, len(payload), token)
        out = protect_packet(self.send, hdr, len(pn), self.next_pn, payload)
        self.next_pn += 1
        return out

    def seal_short(self, dcid: bytes, payload: bytes) -> bytes:
        pn = encode_packet_number(self.next_pn, self.largest_acked)
        payload = payload.ljust(max(len(payload), 4 - len(pn)), b"\0")
        out = protect_packet(self.send, build_short_header(dcid, pn, self.key_phase), len(pn), self.next_pn, payload)
        self.next_pn += 1
        return out

    def initiate_key_update(self) -> None:
        self.send, self.recv = self.send.next_generation(), self.recv.next_generation()
        self.key_phase ^= 1

    def open_long(self, packet: bytes) -> Tuple[dict, int, bytes]:
        info = parse_long_header(packet)
        hdr, pn, payload = unprotect_packet(self.recv, packet[:info["end"]], info["pn_offset"], self.largest_received)
        self.largest_received = max(self.largest_received, pn)
        return info, pn, payload

    def open_short(self, packet: bytes, dcid_len: int) -> Tuple[int, bytes]:
        pn_offset = 1 + dcid_len
        if len(packet) < pn_offset + 20:
            raise ProtectionError("packet too short to sample")
        first = packet[0] ^ (_hp_mask(self.recv, packet[pn_offset + 4:pn_offset + 20])[0] & 0x1F)
        if ((first >> 2) & 1) != self.key_phase:
            nxt = self.recv.next_generation()
            hdr, pn, payload = unprotect_packet(nxt, packet, pn_offset, self.largest_received)   # raises if it is noise
            self.recv, self.send = nxt, self.send.next_generation()
            self.key_phase ^= 1
        else:
            hdr, pn, payload = unprotect_packet(self.recv, packet, pn_offset, self.largest_received)
        self.largest_received = max(self.largest_received, pn)
        return pn, payload
