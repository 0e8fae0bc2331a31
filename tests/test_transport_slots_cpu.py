"""One-sided shared-memory transport, A/B update slots and Montgomery multiplication."""
import multiprocessing as mp
import os

import numpy as np
import pytest

from sneppx_alg_b200.security import crypto, services
from sneppx_alg_b200.utils.net import RDMA


def _peer(key, n):
    r = RDMA()
    r.open()
    buf = np.zeros(n, dtype=np.float32)
    r.read(key, 0, buf)                                   # one-sided read of the owner's region
    r.write(key, 4 * n, (buf * 2).astype(np.float32))     # one-sided write into its second half
    r.close()


def test_one_sided_read_write_between_processes():
    key = f"sxrdma_{os.getpid()}"
    n = 1024
    owner = RDMA()
    owner.open()
    src = np.arange(n, dtype=np.float32)
    view = owner.register_memory(key, array=np.concatenate([src, np.zeros(n, dtype=np.float32)]))
    try:
        p = mp.get_context("spawn").Process(target=_peer, args=(key, n))
        p.start()
        p.join(60)
        assert p.exitcode == 0
        got = view.view(np.float32)
        assert np.array_equal(got[:n], src) and np.array_equal(got[n:], src * 2)
        with pytest.raises(ValueError):
            owner.read(key, 8 * n - 4, np.zeros(4, dtype=np.float32))
        with pytest.raises(ValueError):
            owner.write(key, -1, np.zeros(1, dtype=np.uint8))
    finally:
        del view, got
        owner.close()
    with pytest.raises(FileNotFoundError):
        RDMA().attach(key)                                # the owner's close removed the region


def test_ab_slots_switch_verify_and_rollback(tmp_path):
    slots = services.ABSlots(str(tmp_path))
    assert slots.current == "_a" and slots.inactive_slot == "_b"
    slots.stage("model/weights.bin", b"v2")
    assert not slots.switch_slot(verify=lambda d: False) and slots.current == "_a"
    assert slots.switch_slot(verify=lambda d: open(os.path.join(d, "model/weights.bin"), "rb").read() == b"v2")
    assert slots.current == "_b" and open(slots.get_partition_path("model/weights.bin"), "rb").read() == b"v2"
    assert services.ABSlots(str(tmp_path)).current == "_b"          # the marker survives a restart
    assert slots.rollback() and slots.current == "_a"


def test_montgomery_multiplication():
    p = 2 ** 255 - 19
    m = crypto.MontgomeryMul(p)
    a, b = 0x1234567890ABCDEF ** 3 % p, (p - 12345)
    assert m.from_mont(m.mont_mul(m.to_mont(a), m.to_mont(b))) == a * b % p
    assert m.pow(a, p - 2) == pow(a, p - 2, p) and m.pow(a, p - 2) * a % p == 1
    small = crypto.MontgomeryMul(97)
    assert all(small.from_mont(small.mont_mul(small.to_mont(x), small.to_mont(y))) == x * y % 97 for x in range(97) for y in (0, 1, 50, 96))
    with pytest.raises(ValueError):
        crypto.MontgomeryMul(100)
    assert crypto.MontgomeryMul().mul(3, 4, 7, 1) == 5


def test_secure_multiplexed_streams():
    import threading
    from sneppx_alg_b200.utils.net import FramedSocket, SecureStreamConnection, close_listener
    lfd, port = FramedSocket.listen(0)
    out = {}

    def server():
        c = SecureStreamConnection.accept(lfd, psk=b"cluster-secret")
        out["a"] = c.stream_recv(0)
        big = b""
        while True:
            part = c.stream_recv(2)
            if part is None:
                break
            big += part
        out["big"] = big
        out["b"] = c.stream_recv(0)                       # queued while stream 2 was being drained
        sid = c.stream_open()
        c.stream_send(sid, b"reply on " + str(sid).encode())
        out["server"] = c
    t = threading.Thread(target=server)
    t.start()
    c = SecureStreamConnection.dial("127.0.0.1", port, psk=b"cluster-secret")
    s0, s2 = c.stream_open(), c.stream_open()
    assert (s0, s2) == (0, 2)
    payload = os.urandom(300_000)
    c.stream_send(s0, b"hello")
    c.stream_send(s2, payload[:100_000], chunk=65536)
    c.stream_send(s0, b"second")
    c.stream_send(s2, payload[100_000:], chunk=65536)
    c.stream_close(s2)
    assert c.stream_recv(1) == b"reply on 1"
    t.join(30)
    assert out["a"] == b"hello" and out["b"] == b"second" and out["big"] == payload
    # a frame altered on the wire fails authentication at the receiver
    srv = out["server"]
    c.sock.send_message(b"\x00\x00\x00\x00\x00" + b"x" * 40)
    with pytest.raises(ConnectionError):
        srv.stream_recv(0)
    c.close(); srv.close()

    # a peer with another pre-shared key is turned away during the handshake
    res = {}

    def server2():
        try:
            SecureStreamConnection.accept(lfd, psk=b"cluster-secret")
            res["ok"] = True
        except ConnectionError:
            res["ok"] = False
    t = threading.Thread(target=server2)
    t.start()
    with pytest.raises(ConnectionError):
        SecureStreamConnection.dial("127.0.0.1", port, timeout_ms=2000, psk=b"wrong")
    t.join(30)
    assert res["ok"] is False
    close_listener(lfd)


def test_hybrid_post_quantum_handshake():
    import threading
    from sneppx_alg_b200.utils.net import FramedSocket, SecureStreamConnection, close_listener
    lfd, port = FramedSocket.listen(0)
    out = {}

    def server():
        c = SecureStreamConnection.accept(lfd, post_quantum=True)
        out["msg"] = c.stream_recv(0)
        c.stream_send(c.stream_open(), b"pong")
        out["c"] = c
    t = threading.Thread(target=server)
    t.start()
    c = SecureStreamConnection.dial("127.0.0.1", port, post_quantum=True)
    c.stream_send(c.stream_open(), b"ping")
    assert c.stream_recv(1) == b"pong"
    t.join(30)
    assert out["msg"] == b"ping"
    c.close(); out["c"].close()

    # a classical-only initiator does not get through to a hybrid acceptor
    res = {}

    def server2():
        try:
            SecureStreamConnection.accept(lfd, timeout_ms=2000, post_quantum=True)
            res["ok"] = True
        except ConnectionError:
            res["ok"] = False
    t = threading.Thread(target=server2)
    t.start()
    with pytest.raises(ConnectionError):
        SecureStreamConnection.dial("127.0.0.1", port, timeout_ms=2000)
    t.join(30)
    assert res["ok"] is False
    close_listener(lfd)
