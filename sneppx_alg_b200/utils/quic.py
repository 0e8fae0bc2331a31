"""A QUIC-shaped transport over UDP: encrypted packets with packet numbers, acknowledgements and loss recovery,
a key agreement in the first flight, and independent byte streams multiplexed on one connection.

What it takes from QUIC (RFC 9000 / 9001 / 9002): variable-length integers, long-header packets for the handshake
and short-header packets afterwards, connection ids chosen by each side, CRYPTO / STREAM / ACK / PING /
CONNECTION_CLOSE frames with their RFC layouts, ACK ranges, per-packet AEAD protection with the packet number as
nonce and the header as associated data, initial keys derived from the client's destination connection id,
retransmission of the FRAMES of a lost packet in a new packet (never the packet itself), probe timeouts from a
smoothed RTT, stream reassembly by offset with FIN. What it does not do: TLS 1.3 (the handshake is an ephemeral
X25519 exchange carried in CRYPTO frames, optionally bound to a pre-shared key), header protection, congestion
control beyond a fixed window, migration, 0-RTT. It therefore talks to itself, not to other QUIC stacks.
The wire-exact packet protection of QUIC version 1 (initial secrets, AES-128-GCM / ChaCha20-Poly1305 payload
protection, header protection, Retry tags, key updates) is in ``utils/quic_protection.py``, and the standard handshake
(TLS 1.3 in CRYPTO frames over the three packet-number spaces) in ``utils/quic_tls.py``.

The reference declares this surface as a shell whose functions return 0 / NULL (net/quic/quic_transport.c:30-119:
create_listener / listen / accept / dial / send / recv / stream_open / stream_send / stream_recv / close); the names
below follow it.
"""
from __future__ import annotations

import os
import queue
import socket
import struct
import threading
import time
from typing import Callable, Dict, List, Optional, Tuple

from ..security import crypto

MAX_DATAGRAM = 1200
INITIAL_SALT = bytes.fromhex("38762cf7f55934b34d179ae6a4c80cadccbb7f0a")
F_PADDING, F_PING, F_ACK, F_CRYPTO, F_STREAM, F_CLOSE = 0x00, 0x01, 0x02, 0x06, 0x08, 0x1C


# ----------------------------------------------------------------------------------------------- wire helpers
def encode_varint(v: int) -> bytes:
    if v < 1 << 6:
        return bytes([v])
    if v < 1 << 14:
        return struct.pack(">H", v | 0x4000)
    if v < 1 << 30:
        return struct.pack(">I", v | 0x80000000)
    if v < 1 << 62:
        return struct.pack(">Q", v | 0xC000000000000000)
    raise ValueError("varint out of range")


def decode_varint(buf: bytes, pos: int) -> Tuple[int, int]:
    if pos >= len(buf):
        raise ValueError("truncated varint")
    n = 1 << (buf[pos] >> 6)
    if pos + n > len(buf):
        raise ValueError("truncated varint")
    v = buf[pos] & 0x3F
    for b in buf[pos + 1: pos + n]:
        v = (v << 8) | b
    return v, pos + n


def encode_ack(received: List[int]) -> bytes:
    """ACK frame for a set of received packet numbers (largest first, then gap / range pairs)."""
    pns = sorted(set(received), reverse=True)
    ranges, start, prev = [], pns[0], pns[0]
    for pn in pns[1:]:
        if pn == prev - 1:
            prev = pn
            continue
        ranges.append((start, prev))
        start = prev = pn
    ranges.append((start, prev))
    out = bytes([F_ACK]) + encode_varint(ranges[0][0]) + encode_varint(0) + encode_varint(len(ranges) - 1) + \
        encode_varint(ranges[0][0] - ranges[0][1])
    for (_, lo_prev), (hi, lo) in zip(ranges, ranges[1:]):
        out += encode_varint(lo_prev - hi - 2) + encode_varint(hi - lo)
    return out


def decode_ack(buf: bytes, pos: int) -> Tuple[List[int], int]:
    largest, pos = decode_varint(buf, pos)
    _, pos = decode_varint(buf, pos)
    count, pos = decode_varint(buf, pos)
    first, pos = decode_varint(buf, pos)
    acked = list(range(largest - first, largest + 1))
    lo = largest - first
    for _ in range(count):
        gap, pos = decode_varint(buf, pos)
        rng, pos = decode_varint(buf, pos)
        hi = lo - gap - 2
        lo = hi - rng
        if lo < 0:
            raise ValueError("malformed ACK ranges")
        acked += list(range(lo, hi + 1))
    return acked, pos


class QuicError(RuntimeError):
    pass


# ----------------------------------------------------------------------------------------------- connection
class QuicConnection:
    def __init__(self, endpoint: "QuicEndpoint", peer, local_cid: bytes, remote_cid: bytes, is_client: bool, psk: bytes):
        self.ep, self.peer, self.local_cid, self.remote_cid, self.is_client, self.psk = \
            endpoint, peer, local_cid, remote_cid, is_client, psk
        self.lock = threading.RLock()
        self.established = threading.Event()
        self.closed = False
        self.close_reason = ""
        self.next_pn = 0
        self.sent: Dict[int, Tuple[float, List[bytes], bool]] = {}     # pn -> (time, frames, ack-eliciting)
        self.recv_pns: List[int] = []
        self.largest_recv = -1
        self.ack_pending = False
        self.srtt, self.rttvar = 0.05, 0.025
        self.keys: Optional[Tuple[bytes, bytes]] = None                # (send, recv) 1-RTT keys
        self.init_keys = self._initial_keys(remote_cid if is_client else local_cid)
        self.eph = os.urandom(32)
        self.transcript = b""
        self.stream_send_off: Dict[int, int] = {}
        self._rbuf: Dict[int, Dict[int, bytes]] = {}
        self.stream_read_off: Dict[int, int] = {}
        self.stream_fin: Dict[int, int] = {}
        self.stream_q: Dict[int, "queue.Queue[bytes]"] = {}
        self.next_stream = 0 if is_client else 1
        self.stats = {"packets_sent": 0, "packets_received": 0, "retransmitted_frames": 0, "bytes_sent": 0}

    # ---- keys
    def _initial_keys(self, cid: bytes) -> Tuple[bytes, bytes]:
        secret = crypto.hkdf_sha256(cid, INITIAL_SALT, b"sneppx quic initial", 64)
        c, s = secret[:32], secret[32:]
        return (c, s) if self.is_client else (s, c)

    def _derive(self, peer_pub: bytes) -> None:
        dh = crypto.x25519(self.eph, peer_pub)
        if dh == b"\x00" * 32:
            raise QuicError("low-order key share")
        okm = crypto.hkdf_sha256(dh + self.psk, crypto.sha256(self.transcript), b"sneppx quic 1rtt", 64)
        c, s = okm[:32], okm[32:]
        self.keys = (c, s) if self.is_client else (s, c)

    # ---- packets
    def _seal(self, long_header: bool, frames: List[bytes]) -> bytes:
        pn = self.next_pn
        self.next_pn += 1
        first = 0xC0 if long_header else 0x40
        hdr = bytes([first]) + (bytes([len(self.remote_cid)]) + self.remote_cid + bytes([len(self.local_cid)]) + self.local_cid
                                if long_header else self.remote_cid) + struct.pack(">I", pn)
        key = (self.init_keys if long_header else self.keys)[0]
        payload = b"".join(frames)
        if long_header and len(hdr) + len(payload) + 16 < MAX_DATAGRAM and self.is_client and pn == 0:
            payload += bytes(MAX_DATAGRAM - len(hdr) - len(payload) - 16)      # first flight is padded, as in QUIC
        body = crypto.aead_encrypt(key, b"\x00" * 8 + struct.pack(">I", pn), payload, hdr)
        eliciting = any(f[0] not in (F_ACK, F_PADDING) for f in frames)
        self.sent[pn] = (time.monotonic(), frames, eliciting)
        self.stats["packets_sent"] += 1
        self.stats["bytes_sent"] += len(hdr) + len(body)
        return hdr + body

    def _send_frames(self, frames: List[bytes], long_header: Optional[bool] = None) -> None:
        with self.lock:
            if self.closed and not any(f[0] == F_CLOSE for f in frames):
                raise QuicError(f"connection closed: {self.close_reason}")
            if long_header is None:
                long_header = self.keys is None
            if self.ack_pending and self.recv_pns:
                frames = [encode_ack(self.recv_pns[-64:])] + frames
                self.ack_pending = False
            self.ep._sendto(self._seal(long_header, frames), self.peer)

    # ---- receive path (endpoint thread)
    def _on_packet(self, long_header: bool, pn: int, hdr: bytes, body: bytes) -> None:
        keys = self.init_keys if long_header else self.keys
        if keys is None:
            return
        try:
            payload = crypto.aead_decrypt(keys[1], b"\x00" * 8 + struct.pack(">I", pn), body, hdr)
        except Exception:  # noqa: BLE001  (forged or corrupted packet: dropped silently, as QUIC does)
            return
        with self.lock:
            self.stats["packets_received"] += 1
            if pn in self.recv_pns:
                self.ack_pending = True          # a duplicate means our ACK was lost
            else:
                self.recv_pns.append(pn)
                self.largest_recv = max(self.largest_recv, pn)
                try:
                    self._on_frames(payload)
                except ValueError as e:
                    self._close_local(f"malformed frame: {e}")
                    return
            if self.ack_pending:
                try:
                    self._send_frames([])
                except QuicError:
                    pass

    def _on_frames(self, p: bytes) -> None:
        pos = 0
        while pos < len(p):
            t = p[pos]
            pos += 1
            if t == F_PADDING:
                continue
            if t == F_PING:
                self.ack_pending = True
            elif t in (F_ACK, F_ACK + 1):
                acked, pos = decode_ack(p, pos)
                now = time.monotonic()
                for pn in acked:
                    rec = self.sent.pop(pn, None)
                    if rec and pn == max(acked):
                        sample = now - rec[0]
                        self.rttvar = 0.75 * self.rttvar + 0.25 * abs(self.srtt - sample)
                        self.srtt = 0.875 * self.srtt + 0.125 * sample
            elif t == F_CRYPTO:
                off, pos = decode_varint(p, pos)
                n, pos = decode_varint(p, pos)
                data = p[pos: pos + n]
                pos += n
                self.ack_pending = True
                if len(data) != n or off != 0 or n != 32:
                    raise ValueError("bad CRYPTO frame")
                if self.keys is None:
                    if self.is_client:
                        self.transcript += data
                        self._derive(data)
                    else:
                        self.transcript = data
                        mine = crypto.x25519(self.eph)
                        self.transcript += mine
                        self._derive(data)
                        self.ep._sendto(self._seal(True, [encode_ack(self.recv_pns[-64:]),
                                                          bytes([F_CRYPTO]) + encode_varint(0) + encode_varint(32) + mine]), self.peer)
                        self.ack_pending = False
                    self.established.set()
            elif F_STREAM <= t <= F_STREAM + 7:
                sid, pos = decode_varint(p, pos)
                off = 0
                if t & 0x04:
                    off, pos = decode_varint(p, pos)
                if t & 0x02:
                    n, pos = decode_varint(p, pos)
                else:
                    n = len(p) - pos
                data = p[pos: pos + n]
                pos += n
                if len(data) != n:
                    raise ValueError("truncated STREAM frame")
                self.ack_pending = True
                self._deliver(sid, off, data, bool(t & 0x01))
            elif t == F_CLOSE:
                code, pos = decode_varint(p, pos)
                _, pos = decode_varint(p, pos)
                n, pos = decode_varint(p, pos)
                self._close_local(f"peer closed ({code}): {p[pos: pos + n].decode(errors='replace')}", notify=False)
                return
            else:
                raise ValueError(f"unknown frame type {t:#x}")

    def _deliver(self, sid: int, off: int, data: bytes, fin: bool) -> None:
        buf = self._rbuf.setdefault(sid, {})
        q = self.stream_q.setdefault(sid, queue.Queue())
        if fin:
            self.stream_fin[sid] = off + len(data)
        if data and off >= self.stream_read_off.get(sid, 0):
            buf.setdefault(off, data)
        rd = self.stream_read_off.get(sid, 0)
        while rd in buf:                      # hand contiguous bytes to the reader, in order
            chunk = buf.pop(rd)
            rd += len(chunk)
            q.put(chunk)
        self.stream_read_off[sid] = rd
        if self.stream_fin.get(sid) == rd:
            q.put(b"")                        # end of stream marker
            self.stream_fin[sid] = -1

    # ---- timers (endpoint thread)
    def _on_timer(self, now: float) -> None:
        with self.lock:
            if self.closed:
                return
            pto = max(0.02, self.srtt + 4 * self.rttvar)
            lost = [pn for pn, (t, _, el) in self.sent.items() if el and now - t > pto]
            for pn in lost:
                _, frames, _ = self.sent.pop(pn)
                resend = [f for f in frames if f[0] not in (F_ACK, F_PADDING)]
                if resend:
                    self.stats["retransmitted_frames"] += len(resend)
                    try:
                        self._send_frames(resend, long_header=any(f[0] == F_CRYPTO for f in resend))
                    except QuicError:
                        return
            for pn in [pn for pn, (t, _, el) in self.sent.items() if not el and now - t > 1.0]:
                del self.sent[pn]

    # ---- public API
    def stream_open(self) -> int:
        with self.lock:
            sid = self.next_stream
            self.next_stream += 4          # client-initiated bidirectional streams are 0, 4, 8, ..; server's 1, 5, 9, ..
            self.stream_send_off[sid] = 0
            return sid

    def stream_send(self, sid: int, data: bytes, fin: bool = False) -> None:
        if not self.established.wait(5):
            raise QuicError("handshake did not complete")
        view = memoryview(data)
        chunk = MAX_DATAGRAM - 80
        pos = 0
        while True:
            part = bytes(view[pos: pos + chunk])
            pos += len(part)
            last = pos >= len(data)
            with self.lock:
                off = self.stream_send_off.get(sid, 0)
                self.stream_send_off[sid] = off + len(part)
                while len(self.sent) > 256 and not self.closed:      # fixed window: wait for acknowledgements
                    self.lock.release()
                    time.sleep(0.001)
                    self.lock.acquire()
                t = F_STREAM | 0x04 | 0x02 | (0x01 if (fin and last) else 0)
                self._send_frames([bytes([t]) + encode_varint(sid) + encode_varint(off) + encode_varint(len(part)) + part])
            if last:
                break

    def stream_recv(self, sid: int, timeout: Optional[float] = 5.0) -> bytes:
        """Next chunk of the stream in order; ``b""`` once the peer's FIN has been reached."""
        with self.lock:
            q = self.stream_q.setdefault(sid, queue.Queue())
        try:
            return q.get(timeout=timeout)
        except queue.Empty:
            if self.closed:
                raise QuicError(f"connection closed: {self.close_reason}") from None
            raise TimeoutError("no stream data") from None

    def stream_read_all(self, sid: int, timeout: float = 10.0) -> bytes:
        out, end = b"", time.monotonic() + timeout
        while True:
            chunk = self.stream_recv(sid, max(0.01, end - time.monotonic()))
            if chunk == b"":
                return out
            out += chunk

    def send(self, data: bytes) -> None:
        """Datagram-style convenience on stream 0 / 1 (the connection's default stream)."""
        self.stream_send(0 if self.is_client else 1, struct.pack(">I", len(data)) + data)

    def ping(self) -> None:
        self._send_frames([bytes([F_PING])])

    def _close_local(self, reason: str, notify: bool = True) -> None:
        with self.lock:
            if self.closed:
                return
            if notify and self.keys is not None:
                msg = reason.encode()[:200]
                try:
                    self._send_frames([bytes([F_CLOSE]) + encode_varint(0) + encode_varint(0) + encode_varint(len(msg)) + msg])
                except QuicError:
                    pass
            self.closed, self.close_reason = True, reason
            for q in self.stream_q.values():
                q.put(b"")

    def close(self, reason: str = "closed by application") -> None:
        self._close_local(reason)


class QuicEndpoint:
    """One UDP socket carrying any number of connections (a listener and / or dialler)."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, psk: bytes = b"", drop: Optional[Callable[[bytes], bool]] = None):
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.bind((host, port))
        self.sock.settimeout(0.01)
        self.address = self.sock.getsockname()
        self.psk, self.drop = psk, drop
        self.conns: Dict[bytes, QuicConnection] = {}
        self.accept_q: "queue.Queue[QuicConnection]" = queue.Queue()
        self.listening = False
        self._stop = False
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _sendto(self, datagram: bytes, peer) -> None:
        if self.drop is not None and self.drop(datagram):
            return                                           # test hook: the network lost this datagram
        try:
            self.sock.sendto(datagram, peer)
        except OSError:
            pass

    def _loop(self) -> None:
        last_timer = 0.0
        while not self._stop:
            try:
                data, peer = self.sock.recvfrom(2048)
            except socket.timeout:
                data = None
            except OSError:
                break
            if data:
                try:
                    self._dispatch(data, peer)
                except (ValueError, IndexError, struct.error):
                    pass                                     # malformed datagram: ignored
            now = time.monotonic()
            if now - last_timer > 0.005:
                last_timer = now
                for c in list(self.conns.values()):
                    c._on_timer(now)

    def _dispatch(self, data: bytes, peer) -> None:
        first = data[0]
        if first & 0x80:                                     # long header: dcid len, dcid, scid len, scid, pn
            dl = data[1]
            dcid = data[2: 2 + dl]
            sl = data[2 + dl]
            scid = data[3 + dl: 3 + dl + sl]
            hdr_len = 3 + dl + sl + 4
            pn = struct.unpack(">I", data[hdr_len - 4: hdr_len])[0]
            conn = self.conns.get(dcid)
            if conn is None:
                if not self.listening or len(dcid) != 8 or len(scid) != 8:
                    return
                conn = QuicConnection(self, peer, dcid, scid, False, self.psk)
                self.conns[dcid] = conn
                self.accept_q.put(conn)
            conn._on_packet(True, pn, data[:hdr_len], data[hdr_len:])
        else:
            dcid = data[1:9]
            conn = self.conns.get(dcid)
            if conn is None:
                return
            pn = struct.unpack(">I", data[9:13])[0]
            conn._on_packet(False, pn, data[:13], data[13:])

    # ---- API in the reference's words
    def listen(self) -> None:
        self.listening = True

    def accept(self, timeout: Optional[float] = 5.0) -> QuicConnection:
        try:
            conn = self.accept_q.get(timeout=timeout)
        except queue.Empty:
            raise TimeoutError("no incoming connection") from None
        if not conn.established.wait(timeout):
            raise QuicError("handshake did not complete")
        return conn

    def dial(self, host: str, port: int, timeout: float = 5.0) -> QuicConnection:
        local, remote = os.urandom(8), os.urandom(8)
        conn = QuicConnection(self, (host, port), local, remote, True, self.psk)
        self.conns[local] = conn
        mine = crypto.x25519(conn.eph)
        conn.transcript = mine
        conn._send_frames([bytes([F_CRYPTO]) + encode_varint(0) + encode_varint(32) + mine], long_header=True)
        if not conn.established.wait(timeout):
            conn._close_local("handshake timed out", notify=False)
            raise QuicError("handshake timed out")
        # the server learns our connection id from the long header and answers to it; from now on short headers
        return conn

    def close(self) -> None:
        for c in list(self.conns.values()):
            c.close()
        self._stop = True
        self.thread.join(1)
        self.sock.close()
