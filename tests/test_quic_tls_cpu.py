"""The QUIC v1 handshake: TLS 1.3 in CRYPTO frames over Initial / Handshake / 1-RTT packets, in memory and over UDP."""
import os
import socket

import pytest

from sneppx_alg_b200.security import tls13
from sneppx_alg_b200.utils import quic_protection as qp
from sneppx_alg_b200.utils import quic_tls as qt


@pytest.fixture(scope="module")
def pki():
    seed = os.urandom(32)
    return seed, tls13.make_certificate(seed, "node0.cluster", dns_names=["node0.cluster"])


def exchange(c, s, rounds=6, drop=None):
    """Carry datagrams both ways; ``drop(direction, index)`` may swallow some."""
    n = {"c": 0, "s": 0}
    for _ in range(rounds):
        for src, dst, tag in ((s, c, "s"), (c, s, "c")):
            for d in src.datagrams_to_send():
                n[tag] += 1
                if drop is None or not drop(tag, n[tag]):
                    dst.receive_datagram(d)


def make_pair(pki, store=None, **client_options):
    seed, cert = pki
    opts = dict(server_name="node0.cluster", trusted_roots=[cert])
    opts.update(client_options)
    c = qt.QuicTlsConnection.client(["sx/1"], **opts)
    first = c.datagrams_to_send()
    assert [len(d) for d in first] == [1200]
    s = qt.QuicTlsConnection.accept(first[0], lambda tp: tls13.TlsServer([cert], seed, alpn=["h3", "sx/1"], tickets=store,
                                                                         quic_transport_parameters=tp))
    return c, s


def test_transport_parameters_round_trip():
    p = {qt.TP_ORIGINAL_DCID: b"\x01" * 8, qt.TP_MAX_IDLE_TIMEOUT: 30000, qt.TP_INITIAL_MAX_DATA: 1 << 20, qt.TP_INITIAL_SCID: b""}
    assert qt.decode_transport_parameters(qt.encode_transport_parameters(p)) == p
    with pytest.raises(qt.QuicTlsError):
        qt.decode_transport_parameters(b"\x01\x05\x00")
    assert qt._ack_frame({0, 1, 2, 5, 6, 9}) == bytes([2, 9, 0, 2, 0, 1, 1, 1, 2])


def test_handshake_streams_and_key_discard(pki):
    c, s = make_pair(pki)
    flight = s.datagrams_to_send()
    # the server's first flight is one padded datagram with an Initial and a Handshake packet coalesced
    assert [len(d) for d in flight] == [1200]
    first = qp.parse_long_header(flight[0])
    second = qp.parse_long_header(flight[0][first["end"]:])
    assert (first["type"], second["type"]) == (qp.LONG_INITIAL, qp.LONG_HANDSHAKE) and first["scid"] == s.local_cid
    c.receive_datagram(flight[0])
    assert c.handshake_complete and c.remote_cid == s.local_cid and not c.handshake_confirmed
    exchange(c, s)
    assert s.handshake_complete and c.handshake_confirmed and s.handshake_confirmed
    assert c.tls.alpn == s.tls.alpn == "sx/1" and s.tls.server_name == "node0.cluster"
    assert c.peer_parameters[qt.TP_ORIGINAL_DCID] == c.original_dcid and s.peer_parameters[qt.TP_INITIAL_SCID] == c.local_cid
    for conn in (c, s):
        assert conn.spaces["initial"].discarded and conn.spaces["handshake"].discarded
        assert conn.spaces["application"].protector.send.suite == qp.CHACHA20_POLY1305
    blob = os.urandom(9000)
    c.send_stream(0, blob, fin=True)
    s.send_stream(3, b"server push")
    exchange(c, s)
    assert bytes(s.streams[0]) == blob and 0 in s.finished_streams and bytes(c.streams[3]) == b"server push"
    assert not c.spaces["application"].in_flight and not s.spaces["application"].in_flight       # all acknowledged
    c.update_keys()                                                             # the key-phase bit flips; the server follows
    c.send_stream(8, b"under new keys", fin=True)
    exchange(c, s)
    assert bytes(s.streams[8]) == b"under new keys" and s.spaces["application"].protector.key_phase == 1
    s.send_stream(11, b"and back")
    exchange(c, s)
    assert bytes(c.streams[11]) == b"and back" and not s.spaces["application"].in_flight
    c.close(0, "done")
    exchange(c, s)
    assert s.closed == (0, "done")
    with pytest.raises(qt.QuicTlsError):
        s.send_stream(3, b"late")


def test_lost_and_reordered_datagrams(pki):
    c, s = make_pair(pki)
    exchange(c, s, rounds=3, drop=lambda tag, i: tag == "s" and i == 1)          # the whole first server flight is lost
    assert not c.handshake_complete
    s.on_timeout()
    c.on_timeout()
    exchange(c, s)
    assert c.handshake_confirmed and s.handshake_complete
    data = os.urandom(5000)
    c.send_stream(4, data, fin=True)
    grams = c.datagrams_to_send()
    assert len(grams) > 3
    for d in reversed(grams[1:]):                                                # first one lost, the rest backwards
        s.receive_datagram(d)
    assert 4 not in s.finished_streams
    for d in s.datagrams_to_send():
        c.receive_datagram(d)
    assert len(c.spaces["application"].in_flight) == 1                           # only the lost packet is still owed
    c.on_timeout()
    exchange(c, s)
    assert bytes(s.streams[4]) == data and 4 in s.finished_streams
    # a duplicate and a damaged copy change nothing
    before = bytes(s.streams[4])
    s.receive_datagram(grams[1])
    s.receive_datagram(grams[2][:-1] + bytes([grams[2][-1] ^ 1]))
    assert bytes(s.streams[4]) == before and s.closed is None


def test_psk_resumption_and_aes_suite(pki):
    store = tls13.TicketStore()
    c, s = make_pair(pki, store=store, suites=[tls13.TLS_AES_128_GCM_SHA256])
    exchange(c, s)
    assert c.handshake_confirmed and c.spaces["application"].protector.send.suite == qp.AES_128_GCM
    assert len(c.tls.sessions) == 1                                              # the ticket came in a 1-RTT CRYPTO frame
    c2, s2 = make_pair(pki, store=store, session=c.tls.sessions[0], trusted_roots=[])
    exchange(c2, s2)
    assert c2.handshake_confirmed and c2.tls.used_psk and s2.tls.resumed
    c2.send_stream(0, b"resumed")
    exchange(c2, s2)
    assert bytes(s2.streams[0]) == b"resumed"


def test_failed_authentication_closes_with_a_crypto_error(pki):
    seed, cert = pki
    other = tls13.make_certificate(os.urandom(32), "node0.cluster", dns_names=["node0.cluster"])
    c, s = make_pair(pki, trusted_roots=[other])
    with pytest.raises(qt.QuicTlsError) as e:
        exchange(c, s)
    assert e.value.code == 0x0100 + tls13.ALERT_BAD_CERTIFICATE and c.closed[0] == e.value.code
    for d in c.datagrams_to_send():
        s.receive_datagram(d)
    assert s.closed is not None and s.closed[0] == 0x0100 + tls13.ALERT_BAD_CERTIFICATE
    # a first datagram that is too short, or not version 1, is not a connection attempt
    good = qt.QuicTlsConnection.client(["sx/1"], server_name="x", trusted_roots=[cert]).datagrams_to_send()[0]
    with pytest.raises(qt.QuicTlsError):
        qt.QuicTlsConnection.accept(good[:600], lambda tp: None)
    with pytest.raises(qt.QuicTlsError):
        qt.QuicTlsConnection.accept(good[:1] + b"\x00\x00\x00\x02" + good[5:], lambda tp: None)
    with pytest.raises(ValueError):
        tls13.TlsClient("x", trusted_roots=[cert], quic_transport_parameters=b"")   # QUIC needs ALPN


def test_over_udp_sockets(pki):
    seed, cert = pki
    srv_sock, cli_sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM), socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
    for sk in (srv_sock, cli_sock):
        sk.bind(("127.0.0.1", 0))
        sk.settimeout(5)
    try:
        c = qt.QuicTlsConnection.client(["sx/1"], server_name="node0.cluster", trusted_roots=[cert])
        for d in c.datagrams_to_send():
            cli_sock.sendto(d, srv_sock.getsockname())
        first, peer = srv_sock.recvfrom(2048)
        s = qt.QuicTlsConnection.accept(first, lambda tp: tls13.TlsServer([cert], seed, alpn=["sx/1"], quic_transport_parameters=tp))

        def flush(conn, sock, to):
            n = 0
            for d in conn.datagrams_to_send():
                sock.sendto(d, to)
                n += 1
            return n

        def drain(conn, sock, count):
            for _ in range(count):
                conn.receive_datagram(sock.recvfrom(2048)[0])
        for _ in range(4):
            drain(c, cli_sock, flush(s, srv_sock, peer))
            drain(s, srv_sock, flush(c, cli_sock, srv_sock.getsockname()))
        assert c.handshake_confirmed and s.handshake_complete
        c.send_stream(0, b"gradient bucket 17", fin=True)
        drain(s, srv_sock, flush(c, cli_sock, srv_sock.getsockname()))
        assert bytes(s.streams[0]) == b"gradient bucket 17" and 0 in s.finished_streams
    finally:
        srv_sock.close()
        cli_sock.close()


def test_damaged_input_fails_cleanly(pki):
    """Random damage to the first flights, to certificates and to frames ends in the modules' own error types (or is
    dropped), never in an IndexError or a struct error."""
    import random
    rng = random.Random(7)
    seed, cert = pki

    def mutate(d):
        d = bytearray(d)
        for _ in range(rng.randint(1, 4)):
            k = rng.random()
            if k < 0.5 and d:
                d[rng.randrange(len(d))] = rng.randrange(256)
            elif k < 0.7 and d:
                del d[rng.randrange(len(d)):]
            else:
                d += os.urandom(rng.randint(1, 40))
        return bytes(d)
    make = lambda tp: tls13.TlsServer([cert], seed, alpn=["sx/1"], quic_transport_parameters=tp)
    for it in range(120):
        c = qt.QuicTlsConnection.client(["sx/1"], server_name="node0.cluster", trusted_roots=[cert])
        first = c.datagrams_to_send()[0]
        try:
            if it % 2:
                qt.QuicTlsConnection.accept(mutate(first), make)
            else:
                s = qt.QuicTlsConnection.accept(first, make)
                for d in s.datagrams_to_send():
                    c.receive_datagram(mutate(d))
        except (qt.QuicTlsError, tls13.TlsError):
            pass
    for _ in range(2000):
        try:
            tls13.parse_certificate(mutate(cert))
        except ValueError:
            pass
    for it in range(200):
        c, s = tls13.TlsClient("node0.cluster", trusted_roots=[cert]), tls13.TlsServer([cert], seed, psk_lookup=lambda i: b"k" * 32)
        c.start()
        hello = c.data_to_send()
        try:
            if it % 2:
                s.receive(mutate(hello))
            else:
                s.receive(hello)
                c.receive(mutate(s.data_to_send()))
        except tls13.TlsError:
            pass
    # an authenticated peer that sends a malformed frame gets a FRAME_ENCODING_ERROR close
    c, s = make_pair(pki)
    exchange(c, s)
    c.spaces["application"].queue.append(bytes([0x06, 0x00, 0x40]))          # CRYPTO frame cut off in its length
    with pytest.raises(qt.QuicTlsError) as e:
        exchange(c, s)
    assert e.value.code == 0x07 and s.closed[0] == 0x07
