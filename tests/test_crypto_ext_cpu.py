"""SHA-512, SHA-3 / SHAKE, BLAKE2b, AES-256-GCM and Ed25519 against published vectors and independent implementations."""
import hashlib
import os

import pytest

from sneppx_alg_b200.security import crypto as c

MSGS = [b"", b"abc", b"a" * 71, b"a" * 72, b"a" * 111, b"a" * 112, b"a" * 135, b"a" * 136, b"a" * 137, os.urandom(1000)]


def test_hashes_match_hashlib():
    for m in MSGS:
        assert c.sha512(m) == hashlib.sha512(m).digest()
        assert c.sha3_256(m) == hashlib.sha3_256(m).digest()
        assert c.sha3_512(m) == hashlib.sha3_512(m).digest()
        assert c.shake256(m, 300) == hashlib.shake_256(m).digest(300)
        assert c.blake2b(m) == hashlib.blake2b(m).digest()
        assert c.blake2b(m, 32, key=b"k" * 17) == hashlib.blake2b(m, digest_size=32, key=b"k" * 17).digest()
    with pytest.raises(ValueError):
        c.blake2b(b"x", 65)


def test_aes_gcm_nist_vectors_and_tamper():
    # SP 800-38D test case 14 (256-bit zero key, zero IV, one zero block)
    sealed = c.aes256_gcm_encrypt(bytes(32), bytes(12), bytes(16))
    assert sealed.hex() == "cea7403d4d606b6e074ec5d3baf39d18" + "d0d1c8a799996bf0265b98b5d48ab919"
    # test case 13: empty plaintext
    assert c.aes256_gcm_encrypt(bytes(32), bytes(12), b"").hex() == "530f8afbc74536b9a963b4f1c4cb738b"
    key, iv = bytes(range(32)), bytes(range(12))
    for n in (1, 15, 16, 17, 100):
        pt, aad = os.urandom(n), os.urandom(n % 7)
        s = c.aes256_gcm_encrypt(key, iv, pt, aad)
        assert c.aes256_gcm_decrypt(key, iv, s, aad) == pt
        bad = bytearray(s)
        bad[0] ^= 1
        with pytest.raises(ValueError):
            c.aes256_gcm_decrypt(key, iv, bytes(bad), aad)
        with pytest.raises(ValueError):
            c.aes256_gcm_decrypt(key, iv, s, aad + b"x")


def test_aes_gcm_matches_independent_implementation():
    AESGCM = pytest.importorskip("cryptography.hazmat.primitives.ciphers.aead").AESGCM
    key, iv, pt, aad = os.urandom(32), os.urandom(12), os.urandom(333), os.urandom(20)
    assert c.aes256_gcm_encrypt(key, iv, pt, aad) == AESGCM(key).encrypt(iv, pt, aad)


def test_ed25519_rfc8032_vectors():
    # RFC 8032 section 7.1, tests 1 and 2
    seed = bytes.fromhex("9d61b19deffd5a60ba844af492ec2cc44449c5697b326919703bac031cae7f60")
    pub = bytes.fromhex("d75a980182b10ab7d54bfed3c964073a0ee172f3daa62325af021a68f707511a")
    sig = bytes.fromhex("e5564300c360ac729086e2cc806e828a84877f1eb8e5d974d873e065224901555fb8821590a33bacc61e39701cf9b46b"
                        "d25bf5f0595bbe24655141438e7a100b")
    assert c.ed25519_public_key(seed) == pub and c.ed25519_sign(seed, b"") == sig and c.ed25519_verify(pub, b"", sig)
    seed2 = bytes.fromhex("4ccd089b28ff96da9db6c346ec114e0f5b8a319f35aba624da8cf6ed4fb8a6fb")
    pub2 = bytes.fromhex("3d4017c3e843895a92b70aa74d1b7ebc9c982ccf2ec4968cc0cd55f12af4660c")
    sig2 = bytes.fromhex("92a009a9f0d4cab8720e820b5f642540a2b27b5416503f8fb3762223ebdb69da085ac1e43e15996e458f3613d0f11d8c"
                         "387b2eaeb4302aeeb00d291612bb0c00")
    assert c.ed25519_public_key(seed2) == pub2 and c.ed25519_sign(seed2, b"\x72") == sig2
    assert c.ed25519_verify(pub2, b"\x72", sig2) and not c.ed25519_verify(pub2, b"\x73", sig2)
    assert not c.ed25519_verify(pub, b"\x72", sig2)
    bad = bytearray(sig2)
    bad[40] ^= 1
    assert not c.ed25519_verify(pub2, b"\x72", bytes(bad))
    assert not c.ed25519_verify(pub2, b"\x72", sig2[:32] + b"\xff" * 32)  # S >= L is rejected


def test_ed25519_matches_independent_implementation():
    ed = pytest.importorskip("cryptography.hazmat.primitives.asymmetric.ed25519")
    from cryptography.hazmat.primitives import serialization
    for _ in range(3):
        seed, msg = os.urandom(32), os.urandom(77)
        sk = ed.Ed25519PrivateKey.from_private_bytes(seed)
        pub = sk.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)
        assert c.ed25519_public_key(seed) == pub and c.ed25519_sign(seed, msg) == sk.sign(msg)


def test_signed_update_with_public_key(tmp_path):
    from sneppx_alg_b200.security.services import sign_update, verify_update
    f = tmp_path / "model.bin"
    f.write_bytes(os.urandom(4096))
    seed = os.urandom(32)
    man = sign_update(str(f), seed, "1.4.0", scheme="ed25519")
    pub = c.ed25519_public_key(seed)
    assert verify_update(str(f), man, pub) and not verify_update(str(f), man, pub, min_version="2.0")
    assert not verify_update(str(f), man, c.ed25519_public_key(os.urandom(32)))
    f.write_bytes(b"tampered")
    assert not verify_update(str(f), man, pub)
    man2 = sign_update(str(f), b"shared", "1.0")
    assert verify_update(str(f), man2, b"shared") and not verify_update(str(f), man2, b"other")


def test_schnorr_proof_of_knowledge():
    x = os.urandom(32)
    P = c.schnorr_public(x)
    proof = c.schnorr_prove(x, b"session-42")
    assert c.schnorr_verify(P, proof, b"session-42")
    assert not c.schnorr_verify(P, proof, b"session-43")                       # bound to its context
    assert not c.schnorr_verify(c.schnorr_public(os.urandom(32)), proof, b"session-42")
    bad = bytearray(proof)
    bad[50] ^= 1
    assert not c.schnorr_verify(P, bytes(bad), b"session-42")
    assert c.schnorr_prove(x, b"a") != c.schnorr_prove(x, b"b") and c.schnorr_prove(x, b"a") == c.schnorr_prove(x, b"a")
    # the secret clamped by Ed25519 key expansion gives that key pair's public key: same group, same base point
    import hashlib
    seed = os.urandom(32)
    a = bytearray(hashlib.sha512(seed).digest()[:32])
    a[0] &= 248
    a[31] = (a[31] & 127) | 64
    assert c.schnorr_public(bytes(a)) == c.ed25519_public_key(seed)


def test_argon2id_rfc_vector_and_independent_implementation():
    k = c.argon2id(b"\x01" * 32, b"\x02" * 16, 3, 32, 4, 32, secret=b"\x03" * 8, ad=b"\x04" * 12)
    assert k.hex() == "0d640df58d78766c08c037a34a8b53c9d01ef0452d75b65eb52520e96b01e659"   # RFC 9106 section 5.3
    Argon2id = pytest.importorskip("cryptography.hazmat.primitives.kdf.argon2").Argon2id
    for t, m, p, n in ((1, 8, 1, 16), (2, 64, 2, 32), (3, 100, 3, 80), (1, 256, 4, 200)):
        pwd, salt = os.urandom(13), os.urandom(16)
        want = Argon2id(salt=salt, length=n, iterations=t, lanes=p, memory_cost=m).derive(pwd)
        assert c.argon2id(pwd, salt, t, m, p, n) == want, (t, m, p, n)
    with pytest.raises(ValueError):
        c.argon2id(b"x", b"short", 1, 8, 1)
    with pytest.raises(ValueError):
        c.argon2id(b"x", b"longenoughsalt", 1, 4, 1)


def test_poly1305_rfc_vector():
    key = bytes.fromhex("85d6be7857556d337f4452fe42d506a80103808afb0db2fd4abff6af4149f51b")
    msg = b"Cryptographic Forum Research Group"
    assert c.poly1305(key, msg).hex() == "a8061dc1305136c6c22b8baf0c0127a9"   # RFC 8439 section 2.5.2
    import SneppX_ALG as sx
    assert sx.Poly1305(key).verify(msg, bytes.fromhex("a8061dc1305136c6c22b8baf0c0127a9"))
    a = sx.Argon2(1, 64, 1)
    stored = a.hash(b"pw")
    assert a.verify(b"pw", stored) and not a.verify(b"px", stored)


def test_blake3_against_published_vector_and_independent_implementation():
    assert c.blake3(b"").hex() == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    b3 = pytest.importorskip("blake3")
    key = bytes(range(32))
    for n in (1, 63, 64, 65, 1023, 1024, 1025, 2049, 3073, 5000, 8193, 31744):   # block, chunk and tree boundaries
        m = bytes(i % 251 for i in range(n))
        assert c.blake3(m) == b3.blake3(m).digest()
        assert c.blake3(m, 131) == b3.blake3(m).digest(131)
        assert c.blake3(m, 32, key) == b3.blake3(m, key=key).digest()
    with pytest.raises(ValueError):
        c.blake3(b"x", key=b"short")
