"""TLS 1.3: both roles against each other (certificate, external PSK, resumption, KeyUpdate, ALPN, failures) and against
the OpenSSL command-line programs where they are installed."""
import os
import shutil
import socket
import subprocess
import threading
import time

import pytest

from sneppx_alg_b200.security import tls13 as t

OPENSSL = shutil.which("openssl")
needs_openssl = pytest.mark.skipif(OPENSSL is None, reason="the openssl program is not installed")


def pump(a, b, rounds=12):
    for _ in range(rounds):
        d = a.data_to_send()
        if d:
            b.receive(d)
        d = b.data_to_send()
        if d:
            a.receive(d)


@pytest.fixture(scope="module")
def pki():
    root_seed, seed = os.urandom(32), os.urandom(32)
    root = t.make_certificate(root_seed, "sx test root", ca=True)
    leaf = t.make_certificate(seed, "localhost", issuer_seed=root_seed, issuer="sx test root", dns_names=["localhost", "*.svc.test"])
    return {"root": root, "leaf": leaf, "seed": seed, "root_seed": root_seed}


def test_certificate_round_trip_and_chain_checks(pki):
    p = t.parse_certificate(pki["leaf"])
    assert p["subject"] == "localhost" and p["issuer"] == "sx test root" and p["dns_names"] == ["localhost", "*.svc.test"]
    assert not p["ca"] and t.parse_certificate(pki["root"])["ca"]
    from sneppx_alg_b200.security import crypto
    assert p["public_key"] == crypto.ed25519_public_key(pki["seed"])
    assert t.verify_chain([pki["leaf"]], [pki["root"]], "localhost") == p["public_key"]
    assert t.verify_chain([pki["leaf"], pki["root"]], [pki["root"]], "a.svc.test") == p["public_key"]
    with pytest.raises(t.TlsError, match="do not cover"):
        t.verify_chain([pki["leaf"]], [pki["root"]], "a.b.svc.test")
    with pytest.raises(t.TlsError, match="trusted root"):
        t.verify_chain([pki["leaf"]], [t.make_certificate(os.urandom(32), "sx test root", ca=True)], "localhost")
    with pytest.raises(t.TlsError, match="validity"):
        t.verify_chain([pki["leaf"]], [pki["root"]], "localhost", now=time.time() + 400 * 86400)
    # an intermediate without the CA flag cannot sign
    mid_seed, end_seed = os.urandom(32), os.urandom(32)
    mid = t.make_certificate(mid_seed, "mid", issuer_seed=pki["root_seed"], issuer="sx test root", ca=False)
    end = t.make_certificate(end_seed, "end", issuer_seed=mid_seed, issuer="mid")
    with pytest.raises(t.TlsError, match="broken"):
        t.verify_chain([end, mid], [pki["root"]])
    mid_ca = t.make_certificate(mid_seed, "mid", issuer_seed=pki["root_seed"], issuer="sx test root", ca=True)
    assert t.verify_chain([end, mid_ca], [pki["root"]], "end") == crypto.ed25519_public_key(end_seed)
    tampered = bytearray(pki["leaf"])
    tampered[60] ^= 1
    with pytest.raises((t.TlsError, ValueError)):
        t.verify_chain([bytes(tampered)], [pki["root"]])


@pytest.mark.parametrize("suite", t.SUITES)
def test_certificate_handshake_data_key_update_resumption(pki, suite):
    store = t.TicketStore()
    s = t.TlsServer([pki["leaf"]], pki["seed"], tickets=store, alpn=["h2", "sx/1"])
    c = t.TlsClient("localhost", trusted_roots=[pki["root"]], alpn=["sx/1"], suites=[suite])
    c.start()
    pump(c, s)
    assert c.handshake_complete and s.handshake_complete and c.suite == s.suite == suite
    assert c.alpn == s.alpn == "sx/1" and s.server_name == "localhost" and not c.used_psk
    assert c.peer_public_key == t.parse_certificate(pki["leaf"])["public_key"]
    assert c.export_keying_material("EXPORTER-test", b"ctx") == s.export_keying_material("EXPORTER-test", b"ctx")
    big = os.urandom(70000)                                  # several records
    c.send(big)
    pump(c, s)
    assert s.read() == big
    s.update_keys(request_peer=True)
    s.send(b"after")
    pump(c, s)
    assert c.read() == b"after" and c.key_updates_received == 1 and c.key_updates_sent == 1 and s.key_updates_received == 1
    c.send(b"still works")
    pump(c, s)
    assert s.read() == b"still works"
    c.close()
    pump(c, s)
    assert s.peer_closed
    # resume with the ticket; a ticket works once
    assert len(c.sessions) == 1
    s2, c2 = t.TlsServer([pki["leaf"]], pki["seed"], tickets=store), t.TlsClient("localhost", session=c.sessions[0])
    c2.start()
    pump(c2, s2)
    assert c2.handshake_complete and c2.used_psk and s2.resumed and c2.suite == suite
    s3 = t.TlsServer([pki["leaf"]], pki["seed"], tickets=store)
    c3 = t.TlsClient("localhost", session=c.sessions[0], trusted_roots=[pki["root"]])
    c3.start()
    pump(c3, s3)
    assert c3.handshake_complete and not c3.used_psk and not s3.resumed          # fell back to a full handshake


def test_bytewise_delivery_and_padding(pki):
    s, c = t.TlsServer([pki["leaf"]], pki["seed"]), t.TlsClient("localhost", pinned_keys=[t.parse_certificate(pki["leaf"])["public_key"]])
    c.records.pad_to = 256
    c.start()
    for _ in range(8):
        for src, dst in ((c, s), (s, c)):
            for byte in src.data_to_send():
                dst.receive(bytes([byte]))
    assert c.handshake_complete and s.handshake_complete
    c.send(b"x")
    wire = c.data_to_send()
    assert len(wire) == 5 + 256 + 16                          # one byte of data travels as a 256-byte inner record
    s.receive(wire)
    assert s.read() == b"x"


def test_external_psk_and_failures(pki):
    key = os.urandom(32)
    lookup = lambda ident: key if ident == b"worker-7" else None
    s, c = t.TlsServer(psk_lookup=lookup), t.TlsClient(psk=(b"worker-7", key))
    c.start()
    pump(c, s)
    assert c.handshake_complete and s.handshake_complete and c.used_psk and s.psk_identity == b"worker-7" and not s.resumed
    # wrong key: the binder fails at the server, which answers decrypt_error
    s, c = t.TlsServer(psk_lookup=lookup), t.TlsClient(psk=(b"worker-7", os.urandom(32)))
    c.start()
    with pytest.raises(t.TlsError) as e:
        s.receive(c.data_to_send())
    assert e.value.alert == t.ALERT_DECRYPT_ERROR
    with pytest.raises(t.TlsError) as e:
        c.receive(s.data_to_send())
    assert e.value.received and e.value.alert == t.ALERT_DECRYPT_ERROR
    # unknown identity and no certificate to fall back to
    s, c = t.TlsServer(psk_lookup=lookup), t.TlsClient(psk=(b"stranger", key))
    c.start()
    with pytest.raises(t.TlsError) as e:
        s.receive(c.data_to_send())
    assert e.value.alert == t.ALERT_UNKNOWN_PSK_IDENTITY
    # a server whose certificate is not trusted
    other = t.make_certificate(os.urandom(32), "sx test root", ca=True)
    s, c = t.TlsServer([pki["leaf"]], pki["seed"]), t.TlsClient("localhost", trusted_roots=[other])
    c.start()
    s.receive(c.data_to_send())
    with pytest.raises(t.TlsError) as e:
        c.receive(s.data_to_send())
    assert e.value.alert == t.ALERT_BAD_CERTIFICATE
    # a server that signs with a key other than its certificate's
    s, c = t.TlsServer([pki["leaf"]], os.urandom(32)), t.TlsClient("localhost", trusted_roots=[pki["root"]])
    c.start()
    s.receive(c.data_to_send())
    with pytest.raises(t.TlsError) as e:
        c.receive(s.data_to_send())
    assert e.value.alert == t.ALERT_DECRYPT_ERROR
    # a flipped bit in a protected record
    s, c = t.TlsServer([pki["leaf"]], pki["seed"]), t.TlsClient("localhost", trusted_roots=[pki["root"]])
    c.start()
    pump(c, s)
    c.send(b"payload")
    wire = bytearray(c.data_to_send())
    wire[-3] ^= 0x10
    with pytest.raises(t.TlsError) as e:
        s.receive(bytes(wire))
    assert e.value.alert == t.ALERT_BAD_RECORD_MAC
    with pytest.raises(ValueError):
        t.TlsClient("localhost")                             # nothing to authenticate the server with
    with pytest.raises(t.TlsError):
        t.TlsClient("x", insecure_skip_verify=True).send(b"early")


# --------------------------------------------------------------------------------------------------------- against OpenSSL
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _pem(tmp_path, name, der):
    (tmp_path / f"{name}.der").write_bytes(der)
    subprocess.run([OPENSSL, "x509", "-inform", "DER", "-in", str(tmp_path / f"{name}.der"), "-out", str(tmp_path / f"{name}.pem")],
                   check=True)
    return str(tmp_path / f"{name}.pem")


def _connect_when_ready(port, **opts):
    last = None
    for _ in range(50):
        try:
            return t.connect(("127.0.0.1", port), **opts)
        except ConnectionRefusedError as e:
            last = e
            time.sleep(0.1)
    raise last


def _serve_once(make_server):
    ls = socket.socket()
    ls.bind(("127.0.0.1", 0))
    ls.listen(2)
    result = []

    def run():
        sock, _ = ls.accept()
        sock.settimeout(20)
        try:
            ts = t.TlsSocket(sock, make_server()).handshake()
            data = ts.recv()
            ts.sendall(data.upper())
            result.append((ts.conn.used_psk, data))
            time.sleep(0.3)
            ts.close()
        except Exception as e:                               # reported by the assertion on `result`
            result.append(e)
        finally:
            ls.close()
    th = threading.Thread(target=run, daemon=True)
    th.start()
    return ls.getsockname()[1], th, result


@needs_openssl
def test_openssl_verifies_our_certificates(pki, tmp_path):
    root, leaf = _pem(tmp_path, "root", pki["root"]), _pem(tmp_path, "leaf", pki["leaf"])
    r = subprocess.run([OPENSSL, "verify", "-CAfile", root, "-verify_hostname", "localhost", leaf], capture_output=True, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stderr


@needs_openssl
def test_client_against_openssl_server(tmp_path):
    key, cert = str(tmp_path / "k.pem"), str(tmp_path / "c.pem")
    subprocess.run([OPENSSL, "req", "-x509", "-newkey", "ed25519", "-nodes", "-keyout", key, "-out", cert, "-subj", "/CN=localhost",
                    "-days", "2", "-addext", "subjectAltName=DNS:localhost"], check=True, capture_output=True)
    der = subprocess.run([OPENSSL, "x509", "-in", cert, "-outform", "DER"], check=True, capture_output=True).stdout
    port = _free_port()
    srv = subprocess.Popen([OPENSSL, "s_server", "-accept", f"127.0.0.1:{port}", "-cert", cert, "-key", key, "-tls1_3", "-rev"],
                           stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, stdin=subprocess.PIPE)
    try:
        for suite in t.SUITES:
            s = _connect_when_ready(port, server_name="localhost", trusted_roots=[der], suites=[suite])
            assert s.conn.suite == suite
            s.sendall(b"hello tls\n")
            assert s.recv() == b"slt olleh\n"
            s.conn.update_keys(request_peer=True)             # OpenSSL answers with its own KeyUpdate
            s.sendall(b"after update\n")
            assert s.recv() == b"etadpu retfa\n" and s.conn.key_updates_received == 1
            sessions = s.conn.sessions
            s.close()
            assert sessions, "OpenSSL sends tickets after the handshake"
            s2 = _connect_when_ready(port, server_name="localhost", session=sessions[-1], trusted_roots=[der])
            assert s2.conn.used_psk                           # OpenSSL accepted the resumption binder
            s2.sendall(b"resumed\n")
            assert s2.recv() == b"demuser\n"
            s2.close()
        with pytest.raises(t.TlsError) as e:
            _connect_when_ready(port, server_name="localhost", trusted_roots=[t.make_certificate(os.urandom(32), "localhost")])
        assert e.value.alert == t.ALERT_BAD_CERTIFICATE
    finally:
        srv.terminate()
        srv.wait(10)


@needs_openssl
def test_openssl_client_against_our_server(pki, tmp_path):
    root = _pem(tmp_path, "root", pki["root"])
    port, th, result = _serve_once(lambda: t.TlsServer([pki["leaf"], pki["root"]], pki["seed"]))
    r = subprocess.run([OPENSSL, "s_client", "-connect", f"127.0.0.1:{port}", "-tls1_3", "-CAfile", root, "-verify_return_error",
                        "-servername", "localhost", "-verify_hostname", "localhost", "-quiet"], input=b"hello from openssl\n",
                       capture_output=True, timeout=30)
    th.join(10)
    assert r.returncode == 0 and r.stdout == b"HELLO FROM OPENSSL\n", r.stderr
    assert result == [(False, b"hello from openssl\n")]


@needs_openssl
def test_external_psk_both_ways_with_openssl():
    key = os.urandom(32)
    port, th, result = _serve_once(lambda: t.TlsServer(psk_lookup=lambda i: key if i == b"sx-client" else None))
    r = subprocess.run([OPENSSL, "s_client", "-connect", f"127.0.0.1:{port}", "-tls1_3", "-psk", key.hex(), "-psk_identity", "sx-client",
                        "-quiet"], input=b"psk hello\n", capture_output=True, timeout=30)
    th.join(10)
    assert r.returncode == 0 and r.stdout == b"PSK HELLO\n", r.stderr
    assert result == [(True, b"psk hello\n")]
    port = _free_port()
    srv = subprocess.Popen([OPENSSL, "s_server", "-accept", f"127.0.0.1:{port}", "-nocert", "-psk", key.hex(), "-psk_identity",
                            "sx-client", "-tls1_3", "-rev"], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, stdin=subprocess.PIPE)
    try:
        s = _connect_when_ready(port, psk=(b"sx-client", key))
        assert s.conn.used_psk
        s.sendall(b"abc\n")
        assert s.recv() == b"cba\n"
        s.close()
        with pytest.raises(t.TlsError) as e:
            _connect_when_ready(port, psk=(b"sx-client", os.urandom(32)))
        assert e.value.received
    finally:
        srv.terminate()
        srv.wait(10)
