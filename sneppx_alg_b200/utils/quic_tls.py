"""The QUIC version 1 handshake (RFC 9000 / 9001): TLS 1.3 carried in CRYPTO frames over the three encryption levels.

``QuicTlsConnection`` joins the two wire-exact halves that live elsewhere (``security/tls13.py`` in its QUIC mode, where
handshake messages travel without records and traffic secrets are handed over raw, and ``utils/quic_protection.py`` for
packet protection) into a connection that does no I/O itself: datagrams in through ``receive_datagram``, datagrams out
of ``datagrams_to_send``. It covers

* Initial, Handshake and 1-RTT packet-number spaces with their own keys, ACKs and CRYPTO streams (reassembled by
  offset), coalesced packets in one datagram, padding of datagrams that carry Initial packets to 1200 bytes;
* connection ids: keys for the Initial level from the client's first destination id, the switch to the server's chosen
  id, and authentication of all of them through the transport parameters (original_destination_connection_id,
  initial_source_connection_id), which ride in the TLS extension 57;
* HANDSHAKE_DONE and the discarding of Initial and Handshake keys (RFC 9001 section 4.9), 1-RTT key updates;
* STREAM frames with offsets and FIN once the handshake is complete, CONNECTION_CLOSE, and re-queuing of
  unacknowledged frames on ``on_timeout`` (frames are retransmitted in new packets, never packets).

Left to the caller: timers (call ``on_timeout`` when nothing arrived for a probe interval), flow-control credit beyond
the initial limits advertised here, congestion control, migration, Retry. ``utils/quic.py`` keeps its own lighter
framing; this module is the standards-shaped handshake. The reference's shell (net/quic/quic_transport.c:30-119) has no
handshake to compare with.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Set, Tuple

from ..security import tls13
from ..security.network_ext import TLS_AES_128_GCM_SHA256
from . import quic_protection as qp

LEVELS = ("initial", "handshake", "application")
_LONG_TYPE = {"initial": qp.LONG_INITIAL, "handshake": qp.LONG_HANDSHAKE}
MIN_INITIAL_DATAGRAM = 1200

# transport parameter ids (RFC 9000 section 18.2)
TP_ORIGINAL_DCID, TP_MAX_IDLE_TIMEOUT, TP_MAX_UDP_PAYLOAD, TP_INITIAL_MAX_DATA = 0x00, 0x01, 0x03, 0x04
TP_MAX_STREAM_DATA_BIDI_LOCAL, TP_MAX_STREAM_DATA_BIDI_REMOTE, TP_MAX_STREAM_DATA_UNI = 0x05, 0x06, 0x07
TP_MAX_STREAMS_BIDI, TP_MAX_STREAMS_UNI, TP_INITIAL_SCID = 0x08, 0x09, 0x0F
_BYTES_PARAMS = {TP_ORIGINAL_DCID, TP_INITIAL_SCID, 0x02, 0x10}          # ids, stateless reset token, retry source id

F_PADDING, F_PING, F_ACK, F_ACK_ECN, F_CRYPTO, F_NEW_TOKEN, F_CLOSE, F_CLOSE_APP, F_HANDSHAKE_DONE = 0, 1, 2, 3, 6, 7, 0x1C, 0x1D, 0x1E


class QuicTlsError(RuntimeError):
    def __init__(self, message: str, code: int = 0x0A):                   # PROTOCOL_VIOLATION
        super().__init__(message)
        self.code = code


def encode_transport_parameters(params: Dict[int, object]) -> bytes:
    out = bytearray()
    for pid, value in params.items():
        body = bytes(value) if isinstance(value, (bytes, bytearray)) else qp._varint(int(value))
        out += qp._varint(pid) + qp._varint(len(body)) + body
    return bytes(out)


def decode_transport_parameters(buf: bytes) -> Dict[int, object]:
    out: Dict[int, object] = {}
    pos = 0
    try:
        while pos < len(buf):
            pid, pos = qp._read_varint(buf, pos)
            n, pos = qp._read_varint(buf, pos)
            body = buf[pos:pos + n]
            if len(body) != n or pid in out:
                raise QuicTlsError("malformed transport parameters", 0x08)
            pos += n
            out[pid] = body if pid in _BYTES_PARAMS or not body else qp._read_varint(body, 0)[0]
    except IndexError:
        raise QuicTlsError("malformed transport parameters", 0x08) from None
    return out


def _ack_frame(received: Set[int]) -> bytes:
    pns = sorted(received, reverse=True)
    ranges, start, prev = [], pns[0], pns[0]
    for pn in pns[1:]:
        if pn != prev - 1:
            ranges.append((start, prev))
            start = pn
        prev = pn
    ranges.append((start, prev))
    out = bytearray(qp._varint(F_ACK) + qp._varint(ranges[0][0]) + qp._varint(0) + qp._varint(len(ranges) - 1)
                    + qp._varint(ranges[0][0] - ranges[0][1]))
    for (hi, lo), (phi, plo) in zip(ranges[1:], ranges[:-1]):
        out += qp._varint(plo - hi - 2) + qp._varint(hi - lo)
    return bytes(out)


class _Space:
    """One packet-number space: keys, what was received and still needs acknowledging, the CRYPTO stream in both
    directions, and ack-eliciting frames in flight."""

    def __init__(self):
        self.protector: Optional[qp.PacketProtector] = None
        self.received: Set[int] = set()
        self.ack_needed = False
        self.crypto_send_offset = 0
        self.crypto_recv_next = 0
        self.crypto_recv: Dict[int, bytes] = {}
        self.queue: List[bytes] = []                                       # ack-eliciting frames waiting to be sent
        self.in_flight: Dict[int, List[bytes]] = {}                        # packet number -> the frames it carried
        self.discarded = False


class QuicTlsConnection:
    """One end of a QUIC connection. Build with ``client(...)`` or ``accept(first datagram, ...)``."""

    def __init__(self, is_client: bool, tls: tls13._Connection, local_cid: bytes, remote_cid: bytes, original_dcid: bytes):
        self.is_client, self.tls = is_client, tls
        self.local_cid, self.remote_cid, self.original_dcid = local_cid, remote_cid, original_dcid
        self.spaces = {lvl: _Space() for lvl in LEVELS}
        send, recv = qp.initial_keys(original_dcid, is_client)
        self.spaces["initial"].protector = qp.PacketProtector(send, recv)
        self.handshake_confirmed = False
        self.closed: Optional[Tuple[int, str]] = None
        self.peer_parameters: Dict[int, object] = {}
        self.streams: Dict[int, bytearray] = {}
        self.finished_streams: Set[int] = set()
        self._stream_recv: Dict[int, Dict[int, Tuple[bytes, bool]]] = {}
        self._stream_next: Dict[int, int] = {}
        self._stream_send_offset: Dict[int, int] = {}
        self._done_sent = False
        self._peer_cid_fixed = False
        self._token = b""

    # ------------------------------------------------------------------------------------------------ constructors
    @staticmethod
    def default_parameters() -> Dict[int, object]:
        return {TP_MAX_IDLE_TIMEOUT: 30000, TP_MAX_UDP_PAYLOAD: 1472, TP_INITIAL_MAX_DATA: 1 << 20,
                TP_MAX_STREAM_DATA_BIDI_LOCAL: 1 << 18, TP_MAX_STREAM_DATA_BIDI_REMOTE: 1 << 18, TP_MAX_STREAM_DATA_UNI: 1 << 18,
                TP_MAX_STREAMS_BIDI: 16, TP_MAX_STREAMS_UNI: 16}

    @classmethod
    def client(cls, alpn: List[str], parameters: Optional[Dict[int, object]] = None, **tls_options) -> "QuicTlsConnection":
        """``tls_options`` as for ``tls13.TlsClient`` (server_name, trusted_roots, pinned_keys, psk, session, ...)."""
        local, dcid = os.urandom(8), os.urandom(8)
        params = dict(cls.default_parameters(), **(parameters or {}))
        params[TP_INITIAL_SCID] = local
        tls = tls13.TlsClient(alpn=alpn, quic_transport_parameters=encode_transport_parameters(params), **tls_options)
        conn = cls(True, tls, local, dcid, dcid)
        tls.start()
        conn._pump_tls()
        return conn

    @classmethod
    def accept(cls, first_datagram: bytes, make_tls: Callable[[bytes], tls13.TlsServer],
               parameters: Optional[Dict[int, object]] = None) -> "QuicTlsConnection":
        """Server side, from the first datagram of a new client. ``make_tls(encoded transport parameters)`` returns the
        ``tls13.TlsServer`` for this connection (certificate or PSK, ALPN list, ticket store)."""
        try:
            info = qp.parse_long_header(first_datagram)
        except ValueError as e:
            raise QuicTlsError(f"not a QUIC Initial packet: {e}") from None
        if info["version"] != 1 or info["type"] != qp.LONG_INITIAL:
            raise QuicTlsError("a connection starts with a version 1 Initial packet")
        if len(first_datagram) < MIN_INITIAL_DATAGRAM:
            raise QuicTlsError("Initial datagram shorter than 1200 bytes")
        if len(info["dcid"]) < 8:
            raise QuicTlsError("first destination connection id shorter than 8 bytes")
        local = os.urandom(8)
        params = dict(cls.default_parameters(), **(parameters or {}))
        params[TP_ORIGINAL_DCID], params[TP_INITIAL_SCID] = info["dcid"], local
        conn = cls(False, make_tls(encode_transport_parameters(params)), local, info["scid"], info["dcid"])
        conn.receive_datagram(first_datagram)
        return conn

    # ---------------------------------------------------------------------------------------------------- sending
    def _suite_name(self) -> str:
        return qp.AES_128_GCM if self.tls.suite == TLS_AES_128_GCM_SHA256 else qp.CHACHA20_POLY1305

    def _pump_tls(self) -> None:
        """Move what the TLS machine produced into the spaces: handshake bytes become CRYPTO frames, new secrets become
        packet keys, a finished handshake is announced (server) with HANDSHAKE_DONE."""
        for lvl in LEVELS:
            data = bytes(self.tls.crypto_out[lvl])
            self.tls.crypto_out[lvl].clear()
            sp = self.spaces[lvl]
            for off in range(0, len(data), 1000):
                chunk = data[off:off + 1000]
                sp.queue.append(qp._varint(F_CRYPTO) + qp._varint(sp.crypto_send_offset) + qp._varint(len(chunk)) + chunk)
                sp.crypto_send_offset += len(chunk)
        secrets = self.tls.ks.secrets if self.tls.ks is not None else {}
        mine, theirs = ("c", "s") if self.is_client else ("s", "c")
        for lvl, tag in (("handshake", "hs"), ("application", "ap")):
            sp = self.spaces[lvl]                           # both directions' secrets exist as soon as either is derived
            if sp.protector is None and not sp.discarded and f"{mine} {tag} traffic" in secrets:
                name = self._suite_name()
                sp.protector = qp.PacketProtector(qp.derive_packet_keys(secrets[f"{mine} {tag} traffic"], name),
                                                  qp.derive_packet_keys(secrets[f"{theirs} {tag} traffic"], name))
        if self.tls.handshake_complete:
            if not self.peer_parameters:
                self._check_peer_parameters()
            if not self.is_client and not self._done_sent:
                self._done_sent = True
                self.spaces["application"].queue.append(qp._varint(F_HANDSHAKE_DONE))
                self._confirm()

    def _check_peer_parameters(self) -> None:
        p = decode_transport_parameters(self.tls.peer_quic_parameters)
        if p.get(TP_INITIAL_SCID) != self.remote_cid:
            raise QuicTlsError("initial_source_connection_id does not match the packets", 0x08)
        if self.is_client and p.get(TP_ORIGINAL_DCID) != self.original_dcid:
            raise QuicTlsError("original_destination_connection_id does not match the first packet", 0x08)
        if not self.is_client and TP_ORIGINAL_DCID in p:
            raise QuicTlsError("a client may not send original_destination_connection_id", 0x08)
        self.peer_parameters = p

    def _confirm(self) -> None:
        self.handshake_confirmed = True
        for lvl in ("initial", "handshake"):
            self._discard(lvl)

    def _discard(self, lvl: str) -> None:
        sp = self.spaces[lvl]
        sp.protector, sp.discarded, sp.queue, sp.in_flight, sp.ack_needed = None, True, [], {}, False

    def _seal(self, lvl: str, frames: List[bytes], pad_to: int = 0) -> bytes:
        sp = self.spaces[lvl]
        pr = sp.protector
        pn_bytes = qp.encode_packet_number(pr.next_pn, pr.largest_acked)
        payload = b"".join(frames)
        payload = payload.ljust(max(len(payload), 4 - len(pn_bytes)), b"\0")

        def header(n: int) -> bytes:
            if lvl == "application":
                return qp.build_short_header(self.remote_cid, pn_bytes, pr.key_phase)
            return qp.build_long_header(_LONG_TYPE[lvl], self.remote_cid, self.local_cid, pn_bytes, n,
                                        self._token if lvl == "initial" and self.is_client else b"")
        total = len(header(len(payload))) + len(payload) + qp.TAG_LEN
        if pad_to > total:
            payload += b"\0" * (pad_to - total)                            # PADDING frames
        out = qp.protect_packet(pr.send, header(len(payload)), len(pn_bytes), pr.next_pn, payload)
        pr.next_pn += 1
        return out

    def datagrams_to_send(self) -> List[bytes]:
        """Everything that is ready, as datagrams of at most 1200 bytes: the packets of all levels with something to say
        are coalesced, Initial first; a datagram that carries an Initial packet is padded to exactly 1200."""
        out: List[bytes] = []
        while True:
            budget, plans = MIN_INITIAL_DATAGRAM, []
            for lvl in LEVELS:
                sp = self.spaces[lvl]
                if sp.protector is None or not (sp.queue or sp.ack_needed):
                    continue
                if lvl == "application" and not self.tls.handshake_complete:
                    continue                                               # 1-RTT keys are not used before the handshake ends
                overhead = 1 + 4 + 2 + len(self.remote_cid) + len(self.local_cid) + 1 + len(self._token) + 2 + 4 + qp.TAG_LEN
                frames = [_ack_frame(sp.received)] if sp.ack_needed and sp.received else []
                size, taken = sum(len(f) for f in frames), 0
                while taken < len(sp.queue) and size + len(sp.queue[taken]) + overhead <= budget:
                    size += len(sp.queue[taken])
                    taken += 1
                if not frames and not taken:
                    continue                                               # no room left in this datagram
                plans.append((lvl, frames, taken))
                budget -= size + overhead
            if not plans:
                return out
            packets: Dict[str, bytes] = {}
            for lvl, frames, taken in plans:
                if lvl != "initial":
                    packets[lvl] = self._finish(lvl, frames, taken)
            for lvl, frames, taken in plans:
                if lvl == "initial":
                    rest = sum(len(p) for p in packets.values())
                    packets[lvl] = self._finish(lvl, frames, taken, MIN_INITIAL_DATAGRAM - rest if (self.is_client or taken) else 0)
            if self.is_client and "handshake" in packets and not self.spaces["initial"].discarded:
                self._discard("initial")                                   # RFC 9001 4.9.1: with the first Handshake packet sent
            out.append(b"".join(packets[lvl] for lvl in LEVELS if lvl in packets))

    def _finish(self, lvl: str, frames: List[bytes], taken: int, pad_to: int = 0) -> bytes:
        sp = self.spaces[lvl]
        pn = sp.protector.next_pn
        mine = sp.queue[:taken]
        pkt = self._seal(lvl, frames + mine, pad_to)
        if mine:
            sp.in_flight[pn] = [f for f in mine if f[0] not in (F_CLOSE, F_CLOSE_APP)]
        del sp.queue[:taken]
        sp.ack_needed = False
        return pkt

    def on_timeout(self) -> None:
        """Probe timeout: everything ack-eliciting that is still unacknowledged is queued again (in new packets)."""
        for sp in self.spaces.values():
            if sp.protector is not None:
                for pn in sorted(sp.in_flight):
                    sp.queue.extend(sp.in_flight.pop(pn))

    def send_stream(self, stream_id: int, data: bytes, fin: bool = False) -> None:
        if not self.tls.handshake_complete or self.closed is not None:
            raise QuicTlsError("streams open once the handshake is complete")
        off = self._stream_send_offset.get(stream_id, 0)
        for i in range(0, max(len(data), 1), 1100):
            chunk = data[i:i + 1100]
            last = fin and i + 1100 >= len(data)
            self.spaces["application"].queue.append(bytes([0x0E | (1 if last else 0)]) + qp._varint(stream_id) + qp._varint(off)
                                                    + qp._varint(len(chunk)) + chunk)
            off += len(chunk)
        self._stream_send_offset[stream_id] = off

    def update_keys(self) -> None:
        """Move to the next generation of 1-RTT keys (RFC 9001 section 6); the peer follows when it sees the flipped
        key-phase bit. Allowed once the handshake is confirmed."""
        if not self.handshake_confirmed:
            raise QuicTlsError("a key update needs a confirmed handshake")
        self.spaces["application"].protector.initiate_key_update()

    def close(self, code: int = 0, reason: str = "") -> None:
        if self.closed is None:
            self.closed = (code, reason)
            lvl = next(l for l in reversed(LEVELS) if self.spaces[l].protector is not None
                       and (l != "application" or self.tls.handshake_complete))
            self.spaces[lvl].queue.append(qp._varint(F_CLOSE) + qp._varint(code) + qp._varint(0) + qp._varint(len(reason.encode()))
                                          + reason.encode())

    # -------------------------------------------------------------------------------------------------- receiving
    def receive_datagram(self, datagram: bytes) -> None:
        """Open every packet of the datagram that current keys can open and act on its frames. Packets for discarded or
        not yet available keys, and packets that fail authentication, are dropped silently, as the protocol asks."""
        pos = 0
        while pos < len(datagram) and self.closed is None:
            rest = datagram[pos:]
            if rest[0] & 0x80:
                try:
                    info = qp.parse_long_header(rest)
                except ValueError:
                    return
                if info["version"] != 1 or info["pn_offset"] is None or info["end"] > len(rest) or info["dcid"] not in self._accepted_dcids():
                    return
                lvl = {qp.LONG_INITIAL: "initial", qp.LONG_HANDSHAKE: "handshake"}.get(info["type"])
                pos += info["end"]
                if lvl is None:
                    continue
                self._open(lvl, rest[:info["end"]], info)
            else:
                if rest[0] == 0 and not any(rest):
                    return                                                 # datagram-level padding
                self._open("application", rest, None)
                return

    def _accepted_dcids(self) -> Tuple[bytes, ...]:
        # a server is first addressed by the id the client invented, afterwards by the one it chose
        return (self.local_cid,) if self.is_client else (self.local_cid, self.original_dcid)

    def _open(self, lvl: str, packet: bytes, info: Optional[dict]) -> None:
        sp = self.spaces[lvl]
        if sp.protector is None or (lvl == "application" and not self.tls.handshake_complete):
            return                                                         # 1-RTT data is not read before the handshake ends
        try:
            if info is not None:
                _, pn, payload = sp.protector.open_long(packet)
            else:
                if packet[1:1 + len(self.local_cid)] != self.local_cid:
                    return
                pn, payload = sp.protector.open_short(packet, len(self.local_cid))
        except (qp.ProtectionError, ValueError):
            return
        if pn in sp.received:
            return                                                         # duplicate
        if info is not None:
            if self.is_client and not self._peer_cid_fixed:
                self.remote_cid, self._peer_cid_fixed = info["scid"], True   # the server's own choice replaces the invented id
            elif not self.is_client and lvl == "handshake" and not self.spaces["initial"].discarded:
                self._discard("initial")                                   # RFC 9001 4.9.1: with the first Handshake packet opened
        sp.received.add(pn)
        try:
            if self._frames(lvl, sp, payload):
                sp.ack_needed = True
            self._pump_tls()
        except tls13.TlsError as e:
            self.close(0x0100 + e.alert, str(e))                           # CRYPTO_ERROR range
            raise QuicTlsError(f"handshake failed: {e}", 0x0100 + e.alert) from e
        except QuicTlsError as e:
            self.close(e.code, str(e))
            raise

    def _frames(self, lvl: str, sp: _Space, payload: bytes) -> bool:
        """Act on the frames of one packet; True if any of them asks for an acknowledgement."""
        pos, eliciting = 0, False
        rv = qp._read_varint
        try:
            while pos < len(payload):
                ftype, pos = rv(payload, pos)
                if ftype == F_PADDING:
                    continue
                if ftype in (F_ACK, F_ACK_ECN):
                    largest, pos = rv(payload, pos)
                    _delay, pos = rv(payload, pos)
                    count, pos = rv(payload, pos)
                    first, pos = rv(payload, pos)
                    acked, lo = list(range(largest - first, largest + 1)), largest - first
                    for _ in range(count):
                        gap, pos = rv(payload, pos)
                        length, pos = rv(payload, pos)
                        hi = lo - gap - 2
                        lo = hi - length
                        acked += range(lo, hi + 1)
                    if ftype == F_ACK_ECN:
                        for _ in range(3):
                            _, pos = rv(payload, pos)
                    if largest >= sp.protector.next_pn:
                        raise QuicTlsError("acknowledgement of a packet that was never sent")
                    sp.protector.on_ack(largest)
                    for pn in acked:
                        sp.in_flight.pop(pn, None)
                    continue
                eliciting = True
                if ftype == F_PING:
                    continue
                if ftype == F_CRYPTO:
                    off, pos = rv(payload, pos)
                    n, pos = rv(payload, pos)
                    data = payload[pos:pos + n]
                    if len(data) != n:
                        raise QuicTlsError("truncated CRYPTO frame", 0x07)
                    pos += n
                    if off + n > sp.crypto_recv_next:
                        sp.crypto_recv[off] = data
                    while True:                                            # hand over whatever is now contiguous
                        hit = next((o for o in sp.crypto_recv if o <= sp.crypto_recv_next < o + len(sp.crypto_recv[o])), None)
                        if hit is None:
                            break
                        chunk = sp.crypto_recv.pop(hit)[sp.crypto_recv_next - hit:]
                        sp.crypto_recv_next += len(chunk)
                        self.tls.receive_crypto(lvl, chunk)
                        self._pump_tls()
                elif ftype == F_NEW_TOKEN:
                    n, pos = rv(payload, pos)
                    pos += n
                elif 0x08 <= ftype <= 0x0F:
                    if lvl != "application":
                        raise QuicTlsError("STREAM frame outside 1-RTT packets")
                    sid, pos = rv(payload, pos)
                    off = 0
                    if ftype & 0x04:
                        off, pos = rv(payload, pos)
                    if ftype & 0x02:
                        n, pos = rv(payload, pos)
                    else:
                        n = len(payload) - pos
                    data = payload[pos:pos + n]
                    pos += n
                    self._on_stream(sid, off, data, bool(ftype & 0x01))
                elif ftype == F_HANDSHAKE_DONE:
                    if not self.is_client or lvl != "application":
                        raise QuicTlsError("HANDSHAKE_DONE from a client or outside 1-RTT packets")
                    self._confirm()
                elif ftype in (F_CLOSE, F_CLOSE_APP):
                    code, pos = rv(payload, pos)
                    if ftype == F_CLOSE:
                        _, pos = rv(payload, pos)
                    n, pos = rv(payload, pos)
                    self.closed = (code, payload[pos:pos + n].decode(errors="replace"))
                    return False
                else:
                    raise QuicTlsError(f"frame type {ftype:#x} is not handled here", 0x07)
        except IndexError:
            raise QuicTlsError("truncated frame", 0x07) from None
        return eliciting

    def _on_stream(self, sid: int, off: int, data: bytes, fin: bool) -> None:
        pending = self._stream_recv.setdefault(sid, {})
        nxt = self._stream_next.get(sid, 0)
        if off + len(data) > nxt or (fin and off + len(data) == nxt):
            pending[off] = (data, fin)
        buf = self.streams.setdefault(sid, bytearray())
        while True:
            hit = next((o for o, (d, f) in pending.items() if o <= nxt <= o + len(d)), None)
            if hit is None:
                break
            d, f = pending.pop(hit)
            buf += d[nxt - hit:]
            nxt = hit + len(d)
            if f:
                self.finished_streams.add(sid)
        self._stream_next[sid] = nxt

    @property
    def handshake_complete(self) -> bool:
        return self.tls.handshake_complete
