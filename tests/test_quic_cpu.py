"""QUIC-shaped transport over UDP on loopback: wire helpers, handshake, streams, loss recovery, forged packets."""
import os
import random
import threading

import pytest

from sneppx_alg_b200.utils.quic import QuicEndpoint, QuicError, decode_ack, decode_varint, encode_ack, encode_varint


def test_varints_and_ack_ranges():
    for v in (0, 63, 64, 16383, 16384, (1 << 30) - 1, 1 << 30, (1 << 62) - 1):
        enc = encode_varint(v)
        assert decode_varint(enc, 0) == (v, len(enc)) and len(enc) in (1, 2, 4, 8)
    with pytest.raises(ValueError):
        encode_varint(1 << 62)
    with pytest.raises(ValueError):
        decode_varint(b"\xc0\x00", 0)
    for pns in ([5], [0, 1, 2, 3], [10, 9, 7, 6, 2], [100, 98, 96, 50, 49, 48, 1]):
        frame = encode_ack(pns)
        acked, pos = decode_ack(frame, 1)
        assert sorted(acked) == sorted(pns) and pos == len(frame)


def test_handshake_streams_and_order():
    srv, cli = QuicEndpoint(psk=b"k"), QuicEndpoint(psk=b"k")
    srv.listen()
    got = {}

    def serve():
        c = srv.accept(10)
        got["conn"] = c
        got["a"] = c.stream_read_all(0)
        got["b"] = c.stream_read_all(4)
        s = c.stream_open()
        c.stream_send(s, b"reply:" + got["a"][:5], fin=True)
        got["sid"] = s
    t = threading.Thread(target=serve)
    t.start()
    conn = cli.dial(*srv.address)
    a, b = conn.stream_open(), conn.stream_open()
    assert (a, b) == (0, 4)
    big = os.urandom(300_000)
    conn.stream_send(b, b"second stream", fin=True)      # a small message on another stream does not wait for the big one
    conn.stream_send(a, big, fin=True)
    t.join(30)
    assert got["a"] == big and got["b"] == b"second stream"
    assert conn.stream_read_all(got["sid"]) == b"reply:" + big[:5] and got["sid"] == 1
    conn.close("done")
    srv.close()
    cli.close()


def test_loss_recovery_and_forged_packets():
    rng = random.Random(7)
    dropped = [0]

    def lossy(datagram):
        if rng.random() < 0.2:
            dropped[0] += 1
            return True
        return False
    srv, cli = QuicEndpoint(), QuicEndpoint(drop=lossy)
    srv.drop = lossy
    srv.listen()
    out = {}
    t = threading.Thread(target=lambda: out.update(data=srv.accept(20).stream_read_all(0, timeout=30)))
    t.start()
    conn = cli.dial(*srv.address, timeout=20)
    payload = bytes(range(256)) * 400
    conn.stream_send(conn.stream_open(), payload, fin=True)
    t.join(40)
    assert out["data"] == payload and dropped[0] > 10 and conn.stats["retransmitted_frames"] > 0
    # a forged short-header packet (right connection id, wrong key) is dropped without effect
    cli.sock.sendto(b"\x40" + conn.local_cid + b"\x7f\xff\xff\x00" + os.urandom(40), cli.address)
    cli.sock.sendto(b"\xc0\xff", cli.address)                        # truncated long header
    import time
    time.sleep(0.1)
    assert not conn.closed and 0x7FFFFF00 not in conn.recv_pns            # never accepted: it failed authentication
    srv.close()
    cli.close()


def test_wrong_psk_cannot_talk_and_close_is_seen():
    srv, cli = QuicEndpoint(psk=b"right"), QuicEndpoint(psk=b"wrong")
    srv.listen()
    conn = cli.dial(*srv.address)             # the key shares are exchanged, but the 1-RTT keys differ
    sconn = srv.accept(5)
    conn.stream_send(conn.stream_open(), b"hello", fin=True)
    with pytest.raises(TimeoutError):
        sconn.stream_recv(0, timeout=0.3)     # nothing authentic ever arrives
    srv.close()
    cli.close()
    a, b = QuicEndpoint(), QuicEndpoint()
    a.listen()
    c = b.dial(*a.address)
    sc = a.accept(5)
    c.close("bye")
    import time
    time.sleep(0.2)
    assert sc.closed and "bye" in sc.close_reason
    with pytest.raises(QuicError):
        sc.stream_send(1, b"late")
    a.close()
    b.close()
