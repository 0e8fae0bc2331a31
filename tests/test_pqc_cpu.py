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
