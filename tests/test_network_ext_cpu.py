"""S4 extensions (``security/network_ext.py``): TLS 1.3 key schedule against RFC 8448, Noise handshakes, the tunnel,
block list, intrusion detection, padding, port knocking, RPC credentials, DNS-over-HTTPS messages, certificate
transparency proofs."""
import base64
import hashlib
import hmac
import os
import struct

import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security import network_ext as nx

H = bytes.fromhex


def test_tls13_key_schedule_matches_rfc8448_simple_1rtt():
    ks = nx.Tls13KeySchedule(nx.TLS_AES_128_GCM_SHA256)
    assert ks.early_secret == H("33ad0a1c607ec03b09e6cd9893680ce210adf300aa1f2660e1b22e10f170f92a")
    assert ks.derive_secret(ks.early_secret, "derived", ks.EMPTY_HASH) == \
        H("6f2615a108c702c5678f54fc9dbab69716c076189c48250cebeac3576c3611ba")
    ks.set_shared_secret(H("8bd4054fb55b9d63fdfbacf9f04b9f0d35e6d63f537563efd46272900f89492d"),
                         H("860c06edc07858ee8e78f0e7428c58edd6b43f2ca3e6e95f02ed063cf0e1cad8"))
    assert ks.handshake_secret == H("1dc826e93606aa6fdc0aadc12f741b01046aa6b99f691ed221a9f0ca043fbeac")
    assert ks.secrets["c hs traffic"] == H("b3eddb126e067f35a780b3abf45e2d8f3b1a950738f52e9600746a0e27a55a21")
    assert ks.secrets["s hs traffic"] == H("b67b7d690cc16c4e75e54213cb2d37b4e9c912bcded9105d42befd59d391ad38")
    assert ks.master_secret == H("18df06843d13a08bf2a449844c5f8a478001bc4d4c627984d5a41da8d0402919")
    assert ks.traffic_keys("s hs traffic") == (H("3fce516009c21727d0f2e4e86ee403bc"), H("5d313eb2671276ee13000b30"))
    # the expand step agrees with an HKDF written directly on hashlib
    prk, info = os.urandom(32), b"ctx"
    t1 = hmac.new(prk, info + b"\x01", hashlib.sha256).digest()
    t2 = hmac.new(prk, t1 + info + b"\x02", hashlib.sha256).digest()
    assert nx.hkdf_expand(prk, info, 40) == (t1 + t2)[:40]
    th = hashlib.sha256(b"transcript").digest()
    ks.set_server_finished(th)
    mac = ks.finished_mac("s hs traffic", th)
    assert ks.verify_finished("s hs traffic", th, mac) and not ks.verify_finished("c hs traffic", th, mac)
    before = ks.secrets["c ap traffic"]
    assert ks.update_traffic_secret("c ap traffic") != before and ks.key_generation == 1
    assert len(ks.export_keying_material("EXPORTER-test", b"c", 48)) == 48
    ks.set_client_finished(th)
    assert len(ks.resumption_psk(b"\0\0")) == 32 and ks.binder_key() != ks.binder_key(False)
    assert nx.Tls13KeySchedule.record_nonce(b"\0" * 12, 5)[-1] == 5
    assert nx.negotiate_cipher([0x1302, 0x1301]) == 0x1301 and nx.negotiate_cipher([0x1302]) is None
    assert nx.Tls13KeySchedule(psk=b"k" * 32).early_secret != ks.early_secret
    with pytest.raises(ValueError):
        nx.Tls13KeySchedule(nx.TLS_AES_256_GCM_SHA384)


@pytest.mark.parametrize("pattern", sorted(nx.NOISE_PATTERNS))
def test_noise_handshakes_agree_and_reject_tampering(pattern):
    s_i, s_r = os.urandom(32), os.urandom(32)
    ini = nx.NoiseHandshake(pattern, True, s=s_i, rs=crypto.x25519(s_r), prologue=b"p")
    res = nx.NoiseHandshake(pattern, False, s=s_r, prologue=b"p")
    n = 0
    while not ini.complete:
        w, r = (ini, res) if n % 2 == 0 else (res, ini)
        assert r.read_message(w.write_message(b"payload %d" % n)) == b"payload %d" % n
        n += 1
    assert res.complete and ini.handshake_hash == res.handshake_hash and ini.chaining_key == res.chaining_key
    if pattern in ("XX", "IK"):
        assert res.rs == crypto.x25519(s_i)                                   # the responder learned the initiator's static key
    i2r, r2i = ini.split()
    j2r, s2i = res.split()
    assert j2r.decrypt_with_ad(b"ad", i2r.encrypt_with_ad(b"ad", b"hello")) == b"hello"
    assert r2i.decrypt_with_ad(b"", s2i.encrypt_with_ad(b"", b"back")) == b"back"
    ct = i2r.encrypt_with_ad(b"", b"x")
    with pytest.raises(nx.NoiseError):
        j2r.decrypt_with_ad(b"", ct[:-1] + bytes([ct[-1] ^ 1]))
    i2r.rekey()
    j2r.rekey()
    j2r.n = i2r.n
    assert j2r.decrypt_with_ad(b"", i2r.encrypt_with_ad(b"", b"after rekey")) == b"after rekey"
    # different prologue, or a wrong responder key in a pattern that pre-shares it: the first encrypted part fails
    a = nx.NoiseHandshake(pattern, True, s=s_i, rs=crypto.x25519(s_r), prologue=b"p")
    b = nx.NoiseHandshake(pattern, False, s=s_r, prologue=b"q")
    with pytest.raises(nx.NoiseError):
        m = a.write_message(b"")
        b.read_message(m)
        a.read_message(b.write_message(b""))
        if not a.complete:
            b.read_message(a.write_message(b""))
        raise nx.NoiseError("hashes differ") if a.handshake_hash != b.handshake_hash else AssertionError("prologue ignored")
    with pytest.raises(nx.NoiseError):
        ini2 = nx.NoiseHandshake(pattern, True, s=s_i, rs=crypto.x25519(s_r))
        ini2.read_message(b"")


def test_noise_argument_checks():
    with pytest.raises(ValueError):
        nx.NoiseHandshake("KK", True)
    with pytest.raises(ValueError):
        nx.NoiseHandshake("NK", True)                                         # needs the responder's static key
    with pytest.raises(ValueError):
        nx.NoiseHandshake("XX", True)                                         # sends its own static key
    h = nx.NoiseHandshake("NN", True)
    with pytest.raises(nx.NoiseError):
        h.split()


def test_tunnel_handshake_data_replay_and_rekey():
    now = [1000.0]
    a_priv, b_priv = os.urandom(32), os.urandom(32)
    a = nx.TunnelPeer(a_priv, crypto.x25519(b_priv), clock=lambda: now[0], rekey_after_messages=5)
    b = nx.TunnelPeer(b_priv, clock=lambda: now[0])
    with pytest.raises(nx.TunnelError):
        a.send(b"early")
    a.finish(b.respond(a.initiate(), allowed_peers=[a.public]))
    assert a.established and b.established and b.peer_public == a.public
    pkts = [a.send(b"m%d" % i) for i in range(3)]
    assert b.receive(pkts[2]) == b"m2" and b.receive(pkts[0]) == b"m0"          # out of order inside the window
    with pytest.raises(nx.TunnelError, match="replayed"):
        b.receive(pkts[0])
    bad = pkts[1][:-1] + bytes([pkts[1][-1] ^ 1])
    with pytest.raises(nx.TunnelError, match="authentication"):
        b.receive(bad)
    assert b.receive(pkts[1]) == b"m1" and a.receive(b.keepalive()) == b"" and b.stats()["replays"] == 1
    assert b.stats()["rx_bytes"] == 6 and a.stats()["tx_packets"] == 3
    a.send(b"x")
    a.send(b"y")
    assert a.needs_rekey()
    with pytest.raises(nx.TunnelError, match="used up"):
        a.send(b"z")
    now[0] += 200.0
    with pytest.raises(nx.TunnelError, match="expired"):
        b.receive(pkts[1])
    stranger = nx.TunnelPeer(os.urandom(32), crypto.x25519(b_priv), clock=lambda: now[0])
    with pytest.raises(nx.TunnelError, match="unknown peer"):
        nx.TunnelPeer(b_priv, clock=lambda: now[0]).respond(stranger.initiate(), allowed_peers=[a.public])
    old = nx.TunnelPeer(a_priv, crypto.x25519(b_priv), clock=lambda: now[0] - 1000.0).initiate()
    with pytest.raises(nx.TunnelError, match="stale"):
        nx.TunnelPeer(b_priv, clock=lambda: now[0]).respond(old)
    w = nx.ReplayWindow(size=8)
    assert [w.check_and_update(n) for n in (0, 1, 1, 9, 2, 1, 20, 13, 12)] == [True, True, False, True, True, False, True, True, False]


def test_ip_blocklist():
    bl = nx.IPBlocklist(["10.0.0.0/8", "192.168.1.128/25", "2001:db8::/32", "10.1.0.0/16"])
    assert bl.check("10.1.2.3") and bl.match("10.1.2.3") == "10.0.0.0/8" and not bl.check("192.168.1.5")
    assert bl.match("192.168.1.200") == "192.168.1.128/25" and bl.check("2001:db8::1") and not bl.check("2001:db9::1")
    assert bl.check(int.from_bytes(bytes([10, 9, 9, 9]), "big")) and not bl.add("10.0.0.0/8") and len(bl) == 4
    assert bl.remove("10.0.0.0/8") and not bl.remove("10.0.0.0/8") and bl.check("10.1.2.3") and not bl.check("10.2.0.1")
    assert bl.entries() == ["10.1.0.0/16", "192.168.1.128/25", "2001:db8::/32"]
    bl.add("0.0.0.0/0")
    assert bl.check("8.8.8.8")
    bl.clear()
    assert len(bl) == 0 and not bl.check("8.8.8.8")


def _ipv4(proto, src, dst, body):
    hdr = struct.pack(">BBHHHBBH4s4s", 0x45, 0, 20 + len(body), 0, 0, 64, proto, 0, bytes(src), bytes(dst))
    return hdr + body


def _tcp(sport, dport, flags, payload=b""):
    return struct.pack(">HHIIBBHHH", sport, dport, 0, 0, 5 << 4, flags, 1024, 0, 0) + payload


def test_nids_detectors_and_rules(tmp_path):
    now = [0.0]
    ids = nx.Nids(scan_ports=5, scan_window=2.0, max_icmp_payload=64, clock=lambda: now[0])
    src, dst = (10, 0, 0, 9), (10, 0, 0, 1)
    ok = _ipv4(6, src, dst, _tcp(4000, 80, nx.TCP_ACK | nx.TCP_PSH, b"GET / HTTP/1.1"))
    info = nx.parse_ipv4_packet(ok)
    assert (info.src, info.dport, info.proto, info.payload) == ("10.0.0.9", 80, "tcp", b"GET / HTTP/1.1")
    assert ids.analyze(ok) == [] and nx.parse_ipv4_packet(b"\x45short") is None and ids.analyze(b"junk") == [] and ids.malformed == 1
    kinds = lambda pkt: [a["kind"] for a in ids.analyze(pkt)]          # noqa: E731
    assert kinds(_ipv4(6, src, dst, _tcp(1, 80, 0))) == ["tcp_null_scan"]
    assert kinds(_ipv4(6, src, dst, _tcp(1, 80, nx.TCP_FIN | nx.TCP_PSH | nx.TCP_URG))) == ["tcp_xmas_scan"]
    assert kinds(_ipv4(6, src, dst, _tcp(1, 80, nx.TCP_SYN | nx.TCP_FIN))) == ["tcp_syn_fin"]
    assert kinds(_ipv4(6, src, dst, _tcp(1, 80, nx.TCP_FIN))) == ["tcp_fin_scan"]
    scan = [kinds(_ipv4(6, (10, 0, 0, 7), dst, _tcp(1, 1000 + p, nx.TCP_SYN))) for p in range(5)]
    assert scan[:4] == [[]] * 4 and scan[4] == ["port_scan"]
    slow = []
    for p in range(6):
        now[0] += 1.5
        slow += kinds(_ipv4(6, (10, 0, 0, 8), dst, _tcp(1, 2000 + p, nx.TCP_SYN)))
    assert slow == []                                                          # spread out beyond the window
    assert kinds(_ipv4(1, src, dst, b"\x08\0\0\0\0\0\0\0" + b"A" * 100)) == ["icmp_oversize"]
    ids.add_port_blacklist(23)
    assert ids.should_drop(_ipv4(17, src, dst, struct.pack(">HHHH", 5, 23, 8, 0))) and ids.remove_port_blacklist(23) and \
        not ids.remove_port_blacklist(23)
    r = ids.add_rule('alert tcp any any -> any 80 (msg:"sql injection"; content:"union select"; nocase; sid:1001;)')
    assert (r.dport, r.content, r.nocase, r.sid) == (80, [b"union select"], True, 1001)
    hit = ids.analyze(_ipv4(6, src, dst, _tcp(5, 80, nx.TCP_ACK, b"id=1 UNION SELECT pw")))
    assert [(a["kind"], a["msg"], a["drop"], a["sid"]) for a in hit] == [("rule", "sql injection", False, 1001)]
    assert ids.analyze(_ipv4(6, src, dst, _tcp(5, 8080, nx.TCP_ACK, b"union select"))) == []
    rules = tmp_path / "local.rules"
    rules.write_text('# comment\ndrop udp any any -> any 53 (msg:"bad magic"; content:"|de ad be ef|"; content:"x";)\n')
    assert ids.set_rules(str(rules)) == 1
    assert ids.should_drop(_ipv4(17, src, dst, struct.pack(">HHHH", 5, 53, 13, 0) + b"x\xde\xad\xbe\xef"))
    assert not ids.should_drop(_ipv4(17, src, dst, struct.pack(">HHHH", 5, 53, 12, 0) + b"\xde\xad\xbe\xef"))
    n = ids.alert_count()
    assert n >= 8 and ids.last_alert_time() == now[0]
    ids.clear_alerts()
    assert ids.alert_count() == 0 and ids.last_alert_time() is None
    with pytest.raises(ValueError):
        nx.parse_nids_rule("alert tcp any any any 80 (msg:x;)")


def test_padding_fragmentation_knocking_and_rpc_auth():
    for n in (0, 1, 251, 252, 253, 1000):
        p = nx.traffic_pad(os.urandom(n) if n else b"", 256)
        assert len(p) % 256 == 0 and len(nx.traffic_unpad(p)) == n
    assert len(nx.traffic_pad_to(b"abc", 64)) == 64 and nx.traffic_unpad(nx.traffic_pad_to(b"abc", 64)) == b"abc"
    with pytest.raises(ValueError):
        nx.traffic_pad_to(b"abc", 6)
    with pytest.raises(ValueError):
        nx.traffic_unpad(b"\0\0\0\x01a\x01")
    msg = os.urandom(5000)
    frags = nx.mtu_obfuscate(msg, mtu=600)
    assert {len(f) for f in frags} == {600} and len(frags) >= 9 and nx.mtu_reassemble(reversed(frags)) == msg
    assert nx.mtu_reassemble(nx.mtu_obfuscate(b"", mtu=100, min_fragment=8)) == b""
    with pytest.raises(ValueError):
        nx.mtu_reassemble(frags[1:])
    now = [100.0]
    seq = nx.knock_sequence(b"secret", 4, clock=lambda: now[0])
    assert seq == nx.knock_sequence(b"secret", 4, epoch=3) and seq != nx.knock_sequence(b"secret", 4, epoch=4)
    assert all(20000 <= p < 60000 for p in seq) and nx.port_knock_verify(seq, list(seq)) and not nx.port_knock_verify(seq[:3], seq)
    pk = nx.PortKnock(seq, step_timeout=5.0, open_seconds=30.0, clock=lambda: now[0])
    assert [pk.knock("h", p) for p in seq] == [False, False, False, True] and pk.is_open("h") and not pk.is_open("other")
    now[0] += 31.0
    assert not pk.is_open("h")
    assert not pk.knock("h", seq[0]) and not pk.knock("h", 1) and not pk.knock("h", seq[1])      # a wrong port resets
    pk.knock("g", seq[0])
    now[0] += 6.0
    assert [pk.knock("g", p) for p in seq[1:]] == [False, False, False]                           # too slow: restarted
    auth = nx.GrpcAuth(b"tok-1", grace_s=10.0, clock=lambda: now[0])
    assert auth.verify(b"tok-1") and not auth.verify(b"tok-2") and not auth.verify(b"")
    assert auth.verify_metadata(auth.client_metadata()) and not auth.verify_metadata([("x", "y")])
    new = auth.renew()
    assert auth.verify(new) and auth.verify(b"tok-1") and auth.generation == 2
    now[0] += 11.0
    assert not auth.verify(b"tok-1") and auth.verify(new) and not nx.GrpcAuth().has_token()
    with pytest.raises(RuntimeError):
        nx.GrpcAuth().client_metadata()


def test_dns_over_https_messages_and_cache():
    q = nx.dns_build_query("www.example.com")
    assert q[:2] == b"\0\0" and q[12:] == b"\x03www\x07example\x03com\x00\x00\x01\x00\x01"
    with pytest.raises(ValueError):
        nx.dns_build_query("a..b")

    def answer(query, records):
        body = b""
        for rtype, ttl, rdata in records:
            body += b"\xc0\x0c" + struct.pack(">HHIH", rtype, 1, ttl, len(rdata)) + rdata
        return query[:2] + struct.pack(">HHHHH", 0x8180, 1, len(records), 0, 0) + query[12:] + body

    calls, now = [], [0.0]

    def transport(url, body):
        calls.append((url, body))
        raw = base64.urlsafe_b64decode(url.split("dns=")[1] + "==") if body is None else body
        qtype = struct.unpack(">H", raw[-4:-2])[0]
        if qtype == nx.DNS_A:
            # a CNAME whose target is written with a compression pointer into the question, then two A records
            return answer(raw, [(nx.DNS_CNAME, 300, b"\x03cdn\xc0\x10"), (nx.DNS_A, 60, bytes([93, 184, 216, 34])),
                                (nx.DNS_A, 120, bytes([93, 184, 216, 35]))])
        return answer(raw, [(nx.DNS_AAAA, 30, bytes(15) + b"\x01")])

    r = nx.DohResolver("https://doh.test/dns-query", transport=transport, clock=lambda: now[0])
    assert r.resolve("www.example.com") == ["93.184.216.34", "93.184.216.35"] and "?dns=" in calls[0][0] and calls[0][1] is None
    parsed = nx.dns_parse_response(transport(calls[0][0], None))
    assert parsed["answers"][0]["data"] == "cdn.example.com" and parsed["rcode"] == 0
    assert r.resolve("WWW.example.com.") == ["93.184.216.34", "93.184.216.35"] and (r.queries, r.cache_hits) == (1, 1)
    now[0] += 61.0
    r.resolve("www.example.com")
    assert r.queries == 2 and r.resolve("www.example.com", nx.DNS_AAAA) == ["::1"]
    post = nx.DohResolver("https://doh.test/dns-query", use_post=True, transport=transport)
    assert post.resolve_batch(["www.a.example", "www.b.example"])["www.b.example"][0] == "93.184.216.34" and calls[-1][1] is not None
    nxd = nx.DohResolver("https://doh.test/q", transport=lambda u, b: b"\0\0" + struct.pack(">HHHHH", 0x8183, 0, 0, 0, 0))
    assert nxd.resolve("nope.example") == []
    with pytest.raises(ValueError):
        nx.DohResolver("http://plain.test/")
    with pytest.raises(ValueError):
        nx.dns_parse_response(q)                                               # a query is not a response


def test_certificate_transparency_proofs_and_scts():
    assert nx.ct_merkle_root([]) == hashlib.sha256(b"").digest()
    assert nx.ct_leaf_hash(b"") == H("6e340b9cffb37a989ca544e6bb780a2c78901d3fb33738768511a30617afa01d")
    for n in (1, 2, 3, 5, 8, 13):
        leaves = [b"leaf-%d" % i for i in range(n)]
        root = nx.ct_merkle_root(leaves)
        for i in range(n):
            proof = nx.ct_inclusion_proof(leaves, i)
            assert nx.ct_verify_inclusion(leaves[i], i, n, proof, root)
            assert not nx.ct_verify_inclusion(b"other", i, n, proof, root) and not nx.ct_verify_inclusion(leaves[i], i, n, proof + [root], root)
            if n > 1:
                assert not nx.ct_verify_inclusion(leaves[i], (i + 1) % n, n, proof, root)
        for m in range(1, n + 1):
            cp = nx.ct_consistency_proof(leaves, m)
            old = nx.ct_merkle_root(leaves[:m])
            assert nx.ct_verify_consistency(m, n, old, root, cp)
            if m < n:
                assert not nx.ct_verify_consistency(m, n, old, hashlib.sha256(b"fork").digest(), cp)
    cert = b"0\x82fake-der-certificate"
    seeds = [bytes([i]) * 32 for i in (1, 2, 3)]
    keys = {hashlib.sha256(crypto.ed25519_public_key(s)).digest(): crypto.ed25519_public_key(s) for s in seeds[:2]}
    scts = [nx.ct_issue_sct(cert, s, 1_700_000_000_000 + i, b"ext" if i else b"") for i, s in enumerate(seeds)]
    raw = scts[1].encode()
    back = nx.SignedCertificateTimestamp.parse(raw)
    assert back == scts[1] and back.extensions == b"ext"
    assert nx.ct_verify_sct(raw, cert, keys) and not nx.ct_verify_sct(raw, cert + b"x", keys)
    assert not nx.ct_verify_sct(scts[2], cert, keys)                           # unknown log
    assert not nx.ct_verify_sct(raw, cert, keys, now_ms=1_600_000_000_000)     # dated in the future
    assert not nx.ct_verify_sct(raw[:-3], cert, keys) and not nx.ct_verify_sct(b"short", cert, keys)
    assert nx.ct_verify_all_scts(scts, cert, keys) == (True, [True, True, False])
    assert nx.ct_verify_all_scts([scts[0], scts[0]], cert, keys) == (False, [True, True])        # one log twice is one log
