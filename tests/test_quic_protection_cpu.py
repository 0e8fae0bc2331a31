"""QUIC v1 packet protection against the worked examples of RFC 9001 appendix A, plus round trips, tampering, key
updates and packet-number coding (RFC 9000 appendix A)."""
import os

import pytest

from sneppx_alg_b200.utils import quic_protection as q

H = bytes.fromhex
DCID = H("8394c8f03e515708")
CLIENT_HELLO = H(
    "060040f1010000ed0303ebf8fa56f12939b9584a3896472ec40bb863cfd3e86804fe3a47f06a2b69484c00000413011302010000c0"
    "00000010000e00000b6578616d706c652e636f6dff01000100000a00080006001d0017001800100007000504616c706e0005000501"
    "00000000003300260024001d00209370b2c9caa47fbabaf4559fedba753de171fa71f50f1ce15d43e994ec74d748002b0003020304"
    "000d0010000e0403050306030203080408050806002d00020101001c00024001003900320408ffffffffffffffff05048000ffff07"
    "048000ffff0801100104800075300901100f088394c8f03e51570806048000ffff")
SERVER_FRAMES = H(
    "02000000000600405a020000560303eefce7f7b37ba1d1632e96677825ddf73988cfc79825df566dc5430b9a045a1200130100002e"
    "00330024001d00209d3c940d89690b84d08a60993c144eca684d1081287c834d5311bcf32bb9da1a002b00020304")
SERVER_PACKET = H(
    "cf000000010008f067a5502a4262b5004075c0d95a482cd0991cd25b0aac406a5816b6394100f37a1c69797554780bb38cc5a99f5e"
    "de4cf73c3ec2493a1839b3dbcba3f6ea46c5b7684df3548e7ddeb9c3bf9c73cc3f3bded74b562bfb19fb84022f8ef4cdd93795d77d"
    "06edbb7aaf2f58891850abbdca3d20398c276456cbc42158407dd074ee")


def test_aes128_block_fips197():
    assert q.Aes128(H("000102030405060708090a0b0c0d0e0f")).encrypt_block(H("00112233445566778899aabbccddeeff")) == \
        H("69c4e0d86a7b0430d8cdb78070b4c55a")


def test_aes128_gcm_nist_cases():
    # test cases 1 - 4 of the GCM specification (McGrew & Viega), 128-bit key
    z = b"\0" * 16
    assert q.aes128_gcm_encrypt(z, b"\0" * 12, b"") == H("58e2fccefa7e3061367f1d57a4e7455a")
    assert q.aes128_gcm_encrypt(z, b"\0" * 12, z) == H("0388dace60b6a392f328c2b971b2fe78ab6e47d42cec13bdf53a67b21257bddf")
    key, iv = H("feffe9928665731c6d6a8f9467308308"), H("cafebabefacedbaddecaf888")
    pt = H("d9313225f88406e5a55909c5aff5269a86a7a9531534f7da2e4c303d8a318a721c3c0c95956809532fcf0e2449a6b525"
           "b16aedf5aa0de657ba637b39")
    aad = H("feedfacedeadbeeffeedfacedeadbeefabaddad2")
    sealed = q.aes128_gcm_encrypt(key, iv, pt, aad)
    assert sealed == H("42831ec2217774244b7221b784d0d49ce3aa212f2c02a4e035c17e2329aca12e21d514b25466931c7d8f6a5aac84aa05"
                       "1ba30b396a0aac973d58e0915bc94fbc3221a5db94fae95ae7121a47")
    assert q.aes128_gcm_decrypt(key, iv, sealed, aad) == pt
    with pytest.raises(q.ProtectionError):
        q.aes128_gcm_decrypt(key, iv, sealed, aad[:-1])


def test_initial_secrets_and_keys_rfc9001_a1():
    c, s = q.initial_secrets(DCID)
    assert c == H("c00cf151ca5be075ed0ebfb5c80323c42d6b7db67881289af4008f1f6c357aea")
    assert s == H("3c199828fd139efd216c155ad844cc81fb82fa8d7446fa7d78be803acdda951b")
    ck, sk = q.initial_keys(DCID, is_client=True)
    assert (ck.key, ck.iv, ck.hp) == (H("1f369613dd76d5467730efcbe3b1a22d"), H("fa044b2f42a3fd3b46fb255c"),
                                      H("9f50449e04a0e810283a1e9933adedd2"))
    assert (sk.key, sk.iv, sk.hp) == (H("cf3a5331653c364c88f0f379b6067e37"), H("0ac1493ca1905853b0bba03e"),
                                      H("c206b8d9b9f0f37644430b490eeaa314"))
    sk2, ck2 = q.initial_keys(DCID, is_client=False)
    assert (sk2, ck2) == (sk, ck)


def test_client_initial_rfc9001_a2():
    ck, _ = q.initial_keys(DCID, True)
    hdr = H("c300000001088394c8f03e5157080000449e00000002")
    pkt = q.protect_packet(ck, hdr, 4, 2, CLIENT_HELLO.ljust(1162, b"\0"))
    assert len(pkt) == 1200
    assert pkt[:22] == H("c000000001088394c8f03e5157080000449e7b9aec34")
    assert pkt[22:38] == H("d1b1c98dd7689fb8ec11d242b123dc9b")               # the sample the RFC lists
    assert pkt[-16:] == H("e221af44860018ab0856972e194cd934")
    info = q.parse_long_header(pkt)
    assert info["type"] == q.LONG_INITIAL and info["dcid"] == DCID and info["scid"] == b"" and info["end"] == 1200
    header, pn, payload = q.unprotect_packet(ck, pkt, info["pn_offset"])
    assert header == hdr and pn == 2 and payload.rstrip(b"\0") == CLIENT_HELLO


def test_server_initial_rfc9001_a3():
    _, sk = q.initial_keys(DCID, True)
    hdr = H("c1000000010008f067a5502a4262b50040750001")
    assert q.protect_packet(sk, hdr, 2, 1, SERVER_FRAMES) == SERVER_PACKET
    assert q.build_long_header(q.LONG_INITIAL, b"", H("f067a5502a4262b5"), b"\x00\x01", len(SERVER_FRAMES)) == hdr
    client = q.PacketProtector(*q.initial_keys(DCID, True))
    info, pn, payload = client.open_long(SERVER_PACKET)
    assert pn == 1 and payload == SERVER_FRAMES and info["scid"] == H("f067a5502a4262b5")


def test_retry_rfc9001_a4():
    retry = H("ff000000010008f067a5502a4262b5746f6b656e04a265ba2eff4d829058fb3f0f2496ba")
    assert q.retry_integrity_tag(DCID, retry[:-16]) == retry[-16:]
    assert q.verify_retry(DCID, retry)
    assert not q.verify_retry(DCID[:-1] + b"\x09", retry)
    info = q.parse_long_header(retry)
    assert info["type"] == q.LONG_RETRY and info["token"] == b"token"


def test_chacha20_short_header_rfc9001_a5():
    secret = H("9ac312a7f877468ebe69422748ad00a15443f18203a07d6060f688f30f21632b")
    k = q.derive_packet_keys(secret, q.CHACHA20_POLY1305)
    assert k.key == H("c6d98ff3441c3fe1b2182094f69caa2ed4b716b65488960a7a984979fb23e1c8")
    assert k.iv == H("e0459b3474bdd0e44a41c144")
    assert k.hp == H("25a282b9e82f06f21f488917a4fc8f1b73573685608597d0efcb076b0ab7a7a4")
    assert k.next_generation().secret == H("1223504755036d556342ee9361d253421a826c9ecdf3c7148684b36b714881f9")
    pkt = q.protect_packet(k, H("4200bff4"), 3, 654360564, H("01"))
    assert pkt == H("4cfe4189655e5cd55c41f69080575d7999c25a5bfb")
    header, pn, payload = q.unprotect_packet(k, pkt, 1, largest_pn=654360563)
    assert (header, pn, payload) == (H("4200bff4"), 654360564, H("01"))


def test_packet_number_coding_rfc9000_appendix_a():
    assert q.decode_packet_number(0xA82F30EA, 0x9B32, 16) == 0xA82F9B32
    assert q.encode_packet_number(0xAC5C02, 0xABE8B3) == H("5c02")
    assert q.encode_packet_number(0xACE8FE, 0xABE8B3) == H("ace8fe")
    assert q.encode_packet_number(0) == b"\x00"
    with pytest.raises(ValueError):
        q.encode_packet_number(5, 5)
    for largest, full in ((10, 11), (255, 256), (70000, 70003), (2 ** 40, 2 ** 40 + 90), (300, 290)):
        for nbytes in (1, 2, 4):
            if abs(full - (largest + 1)) < (1 << (8 * nbytes - 1)):
                assert q.decode_packet_number(largest, full & ((1 << (8 * nbytes)) - 1), 8 * nbytes) == full


@pytest.mark.parametrize("suite", [q.AES_128_GCM, q.CHACHA20_POLY1305])
def test_protector_round_trip_tamper_and_key_update(suite):
    c2s, s2c = os.urandom(32), os.urandom(32)
    client = q.PacketProtector(q.derive_packet_keys(c2s, suite), q.derive_packet_keys(s2c, suite))
    server = q.PacketProtector(q.derive_packet_keys(s2c, suite), q.derive_packet_keys(c2s, suite))
    cid = os.urandom(8)
    for i in range(3):
        pkt = client.seal_short(cid, b"\x01")                           # a bare PING is padded up to the sample size
        pn, payload = server.open_short(pkt, len(cid))
        assert pn == i and payload.rstrip(b"\0") == b"\x01"
    client.on_ack(2)
    pkt = client.seal_short(cid, b"stream data " * 20)
    assert (pkt[0] & 0x80) == 0
    bad = bytearray(pkt)
    bad[-1] ^= 1
    with pytest.raises(q.ProtectionError):
        server.open_short(bytes(bad), len(cid))
    assert server.open_short(pkt, len(cid)) == (3, b"stream data " * 20)
    with pytest.raises(q.ProtectionError):
        server.open_short(pkt[:12], len(cid))
    # the client updates its keys; the server follows on the first packet with the new phase and answers in kind
    client.initiate_key_update()
    pn, payload = server.open_short(client.seal_short(cid, b"after update"), len(cid))
    assert payload == b"after update" and server.key_phase == 1
    pn, payload = client.open_short(server.seal_short(cid, b"acknowledged"), len(cid))
    assert payload == b"acknowledged" and client.key_phase == 1
    # a handshake-level long packet between the same pair
    long_pkt = client.seal_long(q.LONG_HANDSHAKE, cid, b"\x01\x02", b"\x06\x00\x05hello")
    info, pn, payload = server.open_long(long_pkt)
    assert info["type"] == q.LONG_HANDSHAKE and info["scid"] == b"\x01\x02" and payload == b"\x06\x00\x05hello"


def test_coalesced_packets_split_by_length():
    keys = q.initial_keys(DCID, True)
    a = q.PacketProtector(*keys)
    first = a.seal_long(q.LONG_INITIAL, DCID, b"\xaa", b"\x06\x00\x02hi", token=b"tok")
    second = a.seal_long(q.LONG_INITIAL, DCID, b"\xaa", b"\x01" + b"\0" * 30)
    datagram = first + second
    b = q.PacketProtector(keys[1], keys[0])
    info, pn, payload = b.open_long(datagram)
    assert (pn, payload, info["token"]) == (0, b"\x06\x00\x02hi", b"tok")
    info2, pn2, payload2 = b.open_long(datagram[info["end"]:])
    assert pn2 == 1 and payload2[0] == 1
