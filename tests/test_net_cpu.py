"""C++ network components: topology routes, framed sockets, coordinator, Raft, health, WebSocket / MQTT codecs.
Failure cases are made on the host (a cut link, a wrong token, a silent peer)."""
import hashlib
import threading

import numpy as np
import pytest

from sneppx_alg_b200.utils import net


def test_topology_routes():
    r = net.Topology.ring(6)
    assert r.next(5) == 0 and r.prev(0) == 5
    assert r.route(0, 2) == [0, 1, 2] and r.route(0, 4) == [0, 5, 4]
    t = net.Topology.tree(7, 2)
    assert t.parent(0) == -1 and t.parent(5) == 2 and t.children(1) == [3, 4] and t.children(3) == []
    assert t.route(3, 6) == [3, 1, 0, 2, 6]
    adj = np.zeros((4, 4), dtype=np.int32)
    adj[0, 1] = adj[1, 2] = 1
    g = net.Topology.graph(adj)
    assert g.route(0, 2) == [0, 1, 2] and g.route(0, 3) is None


def test_framed_socket_messages_and_tensors():
    lfd, port = net.FramedSocket.listen()
    got = {}

    def server():
        s = net.FramedSocket.accept(lfd)
        got["msg"] = s.recv_message()
        got["t"] = s.recv_tensor()
        s.send_message(b"ack")
        s.close()

    th = threading.Thread(target=server)
    th.start()
    c = net.FramedSocket.connect("127.0.0.1", port)
    c.send_message(b"hello \x00 world")
    x = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    c.send_tensor(x)
    assert c.recv_message() == b"ack"
    th.join()
    assert got["msg"] == b"hello \x00 world" and np.array_equal(got["t"], x) and got["t"].dtype == np.float32
    c.set_timeout(200)
    with pytest.raises(ConnectionError):
        c.recv_message()  # the peer has closed
    c.close()
    net.close_listener(lfd)


def test_coordinator_collectives_and_auth():
    srv = net.CoordinatorServer(world=3, token="s3cret")
    try:
        with pytest.raises(PermissionError):
            net.CoordinatorClient("127.0.0.1", srv.port, token="wrong", name="x")
        res = [None] * 3

        def rank_fn(i):
            c = net.CoordinatorClient("127.0.0.1", srv.port, token="s3cret", name=f"node{i}")
            c.barrier()
            parts = c.all_gather(bytes([c.rank]) * 4)
            c.send((c.rank + 1) % 3, b"from%d" % c.rank)
            msg = c.recv((c.rank + 2) % 3)
            c.barrier()
            res[i] = (c.rank, c.world, parts, msg)
            c.close()

        ths = [threading.Thread(target=rank_fn, args=(i,)) for i in range(3)]
        [t.start() for t in ths]
        [t.join(20) for t in ths]
        assert sorted(r[0] for r in res) == [0, 1, 2]
        for rank, world, parts, msg in res:
            assert world == 3 and parts == [bytes([k]) * 4 for k in range(3)]
            assert msg == b"from%d" % ((rank + 2) % 3)
    finally:
        srv.stop()


def test_coordinator_recv_timeout_is_an_error_not_a_hang():
    srv = net.CoordinatorServer(world=1)
    try:
        c = net.CoordinatorClient("127.0.0.1", srv.port, name="solo")
        with pytest.raises(TimeoutError):
            c.recv(0, timeout_ms=100)
        c.barrier()  # connection still usable
        c.close()
    finally:
        srv.stop()


def test_raft_election_replication_and_failover():
    c = net.RaftCluster(5, election_ms=150, heartbeat_ms=50, seed=3)
    c.step(10, 100)
    l1 = c.leader()
    assert l1 >= 0 and sum(c.state(i)["role"] == "leader" for i in range(5)) == 1
    follower = (l1 + 1) % 5
    assert c.propose(follower, b"nope") == -1
    for k in range(3):
        assert c.propose(l1, b"cmd%d" % k) == k + 1
    c.step(10, 20)
    for i in range(5):
        assert c.committed(i) == [b"cmd0", b"cmd1", b"cmd2"]
    # cut the leader off: it keeps accepting entries that can never commit; the rest elect a new leader
    c.set_connected(l1, False)
    c.step(10, 100)
    l2 = c.leader()
    assert l2 >= 0 and l2 != l1 and c.state(l2)["term"] > c.state(l1)["term"]
    assert c.propose(l2, b"cmd3") == 4
    c.step(10, 20)
    # the old leader rejoins with a stale uncommitted entry, which is overwritten by the new leader's log
    c.set_connected(l1, True)
    c.step(10, 60)
    assert c.state(l1)["role"] == "follower"
    for i in range(5):
        assert c.committed(i) == [b"cmd0", b"cmd1", b"cmd2", b"cmd3"]


def test_raft_minority_cannot_commit():
    c = net.RaftCluster(3, seed=1)
    c.step(10, 100)
    l = c.leader()
    for i in range(3):
        if i != l:
            c.set_connected(i, False)
    idx = c.propose(l, b"lost")
    c.step(10, 30)
    assert idx == 1 and c.state(l)["commit_index"] == 0


def test_health_checker():
    h = net.HealthChecker(timeout_ms=1000, max_failures=2)
    assert h.status(7, 0) == "unknown"
    h.report(7, 100, True, 5.0)
    assert h.status(7, 600) == "healthy" and h.status(7, 1200) == "unhealthy"
    h.report(7, 1300, True, 15.0)
    assert h.status(7, 1400) == "healthy" and 5.0 < h.latency(7) < 15.0
    h.report(7, 1500, False)
    h.report(7, 1600, False)
    assert h.status(7, 1700) == "unhealthy"


def test_websocket_and_sha1_vectors():
    assert net.sha1(b"abc") == hashlib.sha1(b"abc").digest()
    assert net.sha1(b"x" * 1000) == hashlib.sha1(b"x" * 1000).digest()
    # RFC 6455 section 1.3 example
    assert net.ws_accept_key("dGhlIHNhbXBsZSBub25jZQ==") == "s3pPLMBiTxaQ9kYGzzhZRbK+xOo="
    # RFC 6455 section 5.7: unmasked and masked "Hello"
    assert net.ws_encode(b"Hello") == bytes([0x81, 0x05]) + b"Hello"
    assert net.ws_encode(b"Hello", mask_key=0x37FA213D) == bytes.fromhex("818537fa213d7f9f4d5158")
    for n in (0, 5, 126, 70000):
        payload = bytes(range(256)) * (n // 256) + bytes(range(n % 256))
        fr = net.ws_encode(payload, opcode=2, mask_key=0xDEADBEEF)
        used, op, fin, out = net.ws_decode(fr + b"extra")
        assert used == len(fr) and op == 2 and fin and out == payload
        assert net.ws_decode(fr[:-1]) is None


def test_mqtt_codec_and_topics():
    assert net.mqtt_connect("c1", 60) == bytes.fromhex("100e00044d5154540402003c00026331")
    p = net.mqtt_publish("a/b", b"x" * 200, qos=1, packet_id=10)
    d = net.mqtt_parse(p)
    assert d["type"] == 3 and d["topic"] == "a/b" and d["qos"] == 1 and d["packet_id"] == 10 and d["payload"] == b"x" * 200
    assert d["header_len"] == 3  # remaining length 207 takes two bytes
    assert net.mqtt_parse(net.mqtt_subscribe("sensors/+/temp", 1, 5))["type"] == 8
    m = net.mqtt_topic_match
    assert m("sport/tennis/+", "sport/tennis/player1") and not m("sport/tennis/+", "sport/tennis/player1/ranking")
    assert m("sport/#", "sport") and m("sport/#", "sport/a/b") and m("#", "a/b") and m("+/+", "/finance")
    assert not m("sport/+", "sport") and m("sport/+", "sport/") and not m("#", "$SYS/x") and m("$SYS/#", "$SYS/x")


def test_service_directory_ttl():
    sd = net.ServiceDirectory()
    sd.register("trainer-0", "_sneppx._tcp", "127.0.0.1", 29500, "rank=0", now_ms=0, ttl_ms=1000)
    sd.register("serve-0", "_http._tcp", "127.0.0.1", 8000, now_ms=0, ttl_ms=5000)
    assert sd.browse("_sneppx._tcp", 500) == [{"name": "trainer-0", "host": "127.0.0.1", "port": 29500, "txt": "rank=0"}]
    assert sd.browse("_sneppx._tcp", 1500) == [] and len(sd.browse("_http._tcp", 1500)) == 1
    assert sd.unregister("serve-0") and not sd.unregister("serve-0")
