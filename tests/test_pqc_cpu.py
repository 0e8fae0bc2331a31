"""ML-KEM (FIPS 203) in the host library against an independent implementation (the `cryptography` package, where its
OpenSSL has ML-KEM) and against the scheme's own properties."""
import hashlib
import os

import pytest

from sneppx_alg_b200.security import crypto


def _oracle():
    try:
        from cryptography.hazmat.primitives.asymmetric import mlkem
        mlkem.MLKEM768PrivateKey.generate()
        return mlkem
    except Exception:
        return None


def test_shake128_matches_hashlib():
    for n in (0, 1, 167, 168, 169, 1000):
        msg = bytes(range(256)) * 4
        assert crypto.shake128(msg[:n], 400) == hashlib.shake_128(msg[:n]).digest(400)


@pytest.mark.parametrize("level", [512, 768, 1024])
def test_mlkem_round_trip_and_implicit_rejection(level):
    ek, dk = crypto.mlkem_keygen(level, seed=bytes(range(64)))
    n_ek, n_dk, n_ct = crypto.mlkem_sizes(level)
    assert (len(ek), len(dk)) == (n_ek, n_dk)
    assert crypto.mlkem_keygen(level, seed=bytes(range(64))) == (ek, dk)          # deterministic in the seed
    for trial in range(4):
        ss, ct = crypto.mlkem_encaps(ek, level, message=bytes([trial]) * 32)
        assert len(ct) == n_ct and len(ss) == 32
        assert crypto.mlkem_decaps(dk, ct, level) == ss
        bad = bytearray(ct)
        bad[trial * 7] ^= 1
        rejected = crypto.mlkem_decaps(dk, bytes(bad), level)
        assert rejected != ss and rejected == crypto.mlkem_decaps(dk, bytes(bad), level)
    # a key whose first coefficient is 0xFFF (>= q) fails the modulus check
    with pytest.raises(ValueError):
        crypto.mlkem_encaps(b"\xff\x0f" + ek[2:], level)
    with pytest.raises(ValueError):
        crypto.mlkem_encaps(ek[:-1], level)


@pytest.mark.parametrize("level", [768, 1024])
def test_mlkem_interoperates_with_independent_implementation(level):
    mlkem = _oracle()
    if mlkem is None:
        pytest.skip("no independent ML-KEM available")
    Priv = getattr(mlkem, f"MLKEM{level}PrivateKey")
    Pub = getattr(mlkem, f"MLKEM{level}PublicKey")
    for trial in range(3):
        seed = os.urandom(64)
        ek, dk = crypto.mlkem_keygen(level, seed=seed)
        theirs = Priv.from_seed_bytes(seed)
        assert theirs.public_key().public_bytes_raw() == ek                        # same key from the same seed
        ss_theirs, ct_theirs = Pub.from_public_bytes(ek).encapsulate()             # they encapsulate, we decapsulate
        assert crypto.mlkem_decaps(dk, ct_theirs, level) == ss_theirs
        ss_ours, ct_ours = crypto.mlkem_encaps(ek, level)                          # we encapsulate, they decapsulate
        assert theirs.decapsulate(ct_ours) == ss_ours
        bad = bytearray(ct_ours)
        bad[5] ^= 0x40
        assert theirs.decapsulate(bytes(bad)) == crypto.mlkem_decaps(dk, bytes(bad), level)   # same rejection secret


def _dsa_oracle():
    try:
        from cryptography.hazmat.primitives.asymmetric import mldsa
        mldsa.MLDSA65PrivateKey.from_seed_bytes(bytes(32))
        return mldsa
    except Exception:
        return None


@pytest.mark.parametrize("level", [44, 65, 87])
def test_mldsa_sign_verify(level):
    pk, sk = crypto.mldsa_keygen(level, seed=bytes(range(32)))
    n_pk, n_sk, n_sig = crypto.mldsa_sizes(level)
    assert (len(pk), len(sk)) == (n_pk, n_sk)
    msg = b"model update 17"
    sig = crypto.mldsa_sign(sk, msg, level, deterministic=True)
    assert len(sig) == n_sig and sig == crypto.mldsa_sign(sk, msg, level, deterministic=True)
    assert crypto.mldsa_sign(sk, msg, level) != sig                                 # hedged signatures differ
    assert crypto.mldsa_verify(pk, msg, sig, level)
    assert crypto.mldsa_verify(pk, msg, crypto.mldsa_sign(sk, msg, level, context=b"ctx"), level, context=b"ctx")
    assert not crypto.mldsa_verify(pk, msg + b"!", sig, level)
    assert not crypto.mldsa_verify(pk, msg, sig, level, context=b"other")
    for pos in (0, 100, n_sig - 1, n_sig - 20):
        bad = bytearray(sig)
        bad[pos] ^= 4
        assert not crypto.mldsa_verify(pk, msg, bytes(bad), level)
    other_pk, _ = crypto.mldsa_keygen(level, seed=bytes(32))
    assert not crypto.mldsa_verify(other_pk, msg, sig, level)


@pytest.mark.parametrize("level", [44, 65, 87])
def test_mldsa_interoperates_with_independent_implementation(level):
    mldsa = _dsa_oracle()
    if mldsa is None:
        pytest.skip("no independent ML-DSA available")
    from cryptography.exceptions import InvalidSignature
    Priv = getattr(mldsa, f"MLDSA{level}PrivateKey")
    Pub = getattr(mldsa, f"MLDSA{level}PublicKey")
    for trial in range(3):
        seed = os.urandom(32)
        pk, sk = crypto.mldsa_keygen(level, seed=seed)
        theirs = Priv.from_seed_bytes(seed)
        assert theirs.public_key().public_bytes_raw() == pk
        msg = os.urandom(50 + trial)
        Pub.from_public_bytes(pk).verify(crypto.mldsa_sign(sk, msg, level), msg)                 # ours -> theirs
        Pub.from_public_bytes(pk).verify(crypto.mldsa_sign(sk, msg, level, context=b"c1"), msg, b"c1")
        assert crypto.mldsa_verify(pk, msg, theirs.sign(msg), level)                              # theirs -> ours
        assert crypto.mldsa_verify(pk, msg, theirs.sign(msg, b"c2"), level, context=b"c2")
        with pytest.raises(InvalidSignature):
            Pub.from_public_bytes(pk).verify(crypto.mldsa_sign(sk, msg, level), msg + b"x")


def test_signed_update_with_post_quantum_signature(tmp_path):
    from sneppx_alg_b200.security import services
    f = tmp_path / "weights.bin"
    f.write_bytes(os.urandom(4096))
    pk, sk = crypto.mldsa_keygen(65)
    manifest = services.sign_update(str(f), sk, "1.4.0", scheme="ml-dsa-65")
    assert services.verify_update(str(f), manifest, pk, min_version="1.0")
    assert not services.verify_update(str(f), manifest, crypto.mldsa_keygen(65)[0])
    spk, ssk = crypto.slhdsa_keygen("128f")
    hashed = services.sign_update(str(f), ssk, "1.4.0", scheme="slh-dsa-128f")
    assert services.verify_update(str(f), hashed, spk) and not services.verify_update(str(f), hashed, crypto.slhdsa_keygen("128f")[0])
    f.write_bytes(b"tampered")
    assert not services.verify_update(str(f), manifest, pk) and not services.verify_update(str(f), hashed, spk)


def test_hybrid_key_exchange_x25519_mlkem():
    """X25519 + ML-KEM-768 secrets combined through HKDF: both sides derive the same session key."""
    a_x = os.urandom(32)
    b_x = os.urandom(32)
    ek, dk = crypto.mlkem_keygen(768)
    ss_b, ct = crypto.mlkem_encaps(ek, 768)
    key_b = crypto.hkdf_sha256(crypto.x25519(b_x, crypto.x25519(a_x)) + ss_b, info=b"hybrid")
    key_a = crypto.hkdf_sha256(crypto.x25519(a_x, crypto.x25519(b_x)) + crypto.mlkem_decaps(dk, ct, 768), info=b"hybrid")
    assert key_a == key_b


def test_slhdsa_128f_sign_verify():
    pk, sk = crypto.slhdsa_keygen("128f", seed=bytes(range(48)))
    assert crypto.slhdsa_sizes("128f") == (32, 64, 17088) and crypto.slhdsa_sizes("128s") == (32, 64, 7856)
    assert (len(pk), len(sk)) == (32, 64) and sk[32:] == pk and sk[:48] == bytes(range(48))
    msg = b"checkpoint 000123"
    sig = crypto.slhdsa_sign(sk, msg, deterministic=True)
    assert len(sig) == 17088 and sig == crypto.slhdsa_sign(sk, msg, deterministic=True)
    assert crypto.slhdsa_verify(pk, msg, sig)
    hedged = crypto.slhdsa_sign(sk, msg, context=b"ctx")
    assert hedged != sig and crypto.slhdsa_verify(pk, msg, hedged, context=b"ctx")
    assert not crypto.slhdsa_verify(pk, msg, hedged)                               # wrong context
    assert not crypto.slhdsa_verify(pk, msg + b".", sig)
    # one changed byte in the randomiser, a FORS secret, a FORS path, a WOTS chain value or an XMSS path
    for pos in (0, 16, 16 + 40, 16 + 33 * 7 * 16 + 5, 17088 - 1):
        bad = bytearray(sig)
        bad[pos] ^= 1
        assert not crypto.slhdsa_verify(pk, msg, bytes(bad))
    other_pk, _ = crypto.slhdsa_keygen("128f")
    assert not crypto.slhdsa_verify(other_pk, msg, sig)


def test_reference_shaped_classes():
    kem = crypto.KyberKEM(768)
    pk, sk = kem.keypair()
    ct, ss = kem.encapsulate(pk)
    assert kem.decapsulate(sk, ct) == ss and kem.keypair(b"seed") == kem.keypair(b"seed")
    dsa = crypto.Dilithium(crypto.Dilithium.MODE_ML_DSA_65)
    pk, sk = dsa.keypair(b"seed")
    assert dsa.verify(pk, b"m", dsa.sign(sk, b"m")) and not dsa.verify(pk, b"n", dsa.sign(sk, b"m"))
    sp = crypto.SphincsPlus()
    pk, sk = sp.keypair(b"seed")
    assert sp.verify(pk, b"m", sp.sign(sk, b"m"))
