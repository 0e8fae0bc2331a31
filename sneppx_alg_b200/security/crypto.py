"""S0 crypto bindings (``csrc/host/crypto.cpp``): hashes, MACs, KDFs, ChaCha20-Poly1305 AEAD, SipHash, X25519,
HMAC-DRBG, constant-time compare, guarded allocations."""
from __future__ import annotations

import ctypes as C
import os

from .. import _build


def _L():
    L = _build.load_host()
    if not getattr(L, "_crypto_ready", False):
        L.sx_siphash24.restype = C.c_uint64
        L.sx_guarded_alloc.restype = C.c_void_p
        L.sx_guarded_alloc.argtypes = [C.c_size_t]
        L.sx_guarded_check.argtypes = L.sx_guarded_free.argtypes = [C.c_void_p]
        L._crypto_ready = True
    return L


def _buf(n):
    return C.create_string_buffer(n)


def sha256(data: bytes) -> bytes:
    out = _buf(32)
    _L().sx_sha256(data, C.c_size_t(len(data)), out)
    return out.raw


def hmac_sha256(key: bytes, msg: bytes) -> bytes:
    out = _buf(32)
    _L().sx_hmac_sha256(key, C.c_size_t(len(key)), msg, C.c_size_t(len(msg)), out)
    return out.raw


def hkdf_sha256(ikm: bytes, salt: bytes = b"", info: bytes = b"", length: int = 32) -> bytes:
    out = _buf(length)
    _L().sx_hkdf_sha256(ikm, C.c_size_t(len(ikm)), salt, C.c_size_t(len(salt)), info, C.c_size_t(len(info)), out, C.c_size_t(length))
    return out.raw


def pbkdf2_sha256(password: bytes, salt: bytes, iterations: int, length: int = 32) -> bytes:
    out = _buf(length)
    _L().sx_pbkdf2_sha256(password, C.c_size_t(len(password)), salt, C.c_size_t(len(salt)), iterations, out, C.c_size_t(length))
    return out.raw


def chacha20(key: bytes, nonce: bytes, data: bytes, counter: int = 0) -> bytes:
    out = _buf(len(data))
    _L().sx_chacha20(key, C.c_uint32(counter), nonce, data, out, C.c_size_t(len(data)))
    return out.raw


def aead_encrypt(key: bytes, nonce: bytes, plaintext: bytes, aad: bytes = b"") -> bytes:
    """ChaCha20-Poly1305 (RFC 8439): returns ciphertext || 16-byte tag."""
    ct, tag = _buf(len(plaintext)), _buf(16)
    _L().sx_aead_encrypt(key, nonce, aad, C.c_size_t(len(aad)), plaintext, C.c_size_t(len(plaintext)), ct, tag)
    return ct.raw + tag.raw


def aead_decrypt(key: bytes, nonce: bytes, sealed: bytes, aad: bytes = b"") -> bytes:
    ct, tag = sealed[:-16], sealed[-16:]
    pt = _buf(len(ct))
    if _L().sx_aead_decrypt(key, nonce, aad, C.c_size_t(len(aad)), ct, C.c_size_t(len(ct)), tag, pt) != 0:
        raise ValueError("authentication failed")
    return pt.raw


def siphash24(key: bytes, msg: bytes) -> int:
    return _L().sx_siphash24(key, msg, C.c_size_t(len(msg)))


def x25519(scalar: bytes, point: bytes = None) -> bytes:
    out = _buf(32)
    if point is None:
        _L().sx_x25519_base(out, scalar)
    else:
        _L().sx_x25519(out, scalar, point)
    return out.raw


def ct_equal(a: bytes, b: bytes) -> bool:
    return len(a) == len(b) and bool(_L().sx_ct_equal(a, b, C.c_size_t(len(a))))


class HmacDrbg:
    def __init__(self, seed: bytes = None):
        self.state = _buf(64)
        seed = seed if seed is not None else os.urandom(48)
        _L().sx_drbg_init(self.state, seed, C.c_size_t(len(seed)))

    def generate(self, n: int) -> bytes:
        out = _buf(n)
        _L().sx_drbg_generate(self.state, out, C.c_size_t(n))
        return out.raw


class GuardedBuffer:
    """S1: heap block fenced by canaries; ``check`` reports overruns, ``free`` wipes the contents."""

    def __init__(self, n: int):
        self.n = n
        self.ptr = _L().sx_guarded_alloc(n)

    def write(self, data: bytes, offset: int = 0):
        C.memmove(self.ptr + offset, data, len(data))

    def read(self) -> bytes:
        return C.string_at(self.ptr, self.n)

    def check(self) -> int:
        return _L().sx_guarded_check(self.ptr)

    def free(self) -> int:
        rc = _L().sx_guarded_free(self.ptr)
        self.ptr = None
        return rc


# ------------------------------------------------------------------------------- csrc/host/crypto_ext.cpp
def _hash(fn, data: bytes, n: int) -> bytes:
    out = _buf(n)
    getattr(_L(), fn)(data, C.c_size_t(len(data)), out)
    return out.raw


def sha512(data: bytes) -> bytes:
    return _hash("sx_sha512", data, 64)


def sha3_256(data: bytes) -> bytes:
    return _hash("sx_sha3_256", data, 32)


def sha3_512(data: bytes) -> bytes:
    return _hash("sx_sha3_512", data, 64)


def shake256(data: bytes, length: int) -> bytes:
    out = _buf(length)
    _L().sx_shake256(data, C.c_size_t(len(data)), out, C.c_size_t(length))
    return out.raw


def blake2b(data: bytes, digest_size: int = 64, key: bytes = b"") -> bytes:
    out = _buf(digest_size)
    if _L().sx_blake2b(data, C.c_size_t(len(data)), key, C.c_size_t(len(key)), out, C.c_size_t(digest_size)):
        raise ValueError("digest_size must be 1..64 and the key at most 64 bytes")
    return out.raw


def aes256_gcm_encrypt(key: bytes, iv: bytes, plaintext: bytes, aad: bytes = b"") -> bytes:
    """AES-256-GCM with a 96-bit IV: returns ciphertext || 16-byte tag."""
    if len(key) != 32 or len(iv) != 12:
        raise ValueError("key must be 32 bytes and iv 12 bytes")
    ct, tag = _buf(max(len(plaintext), 1)), _buf(16)
    _L().sx_aes256_gcm_encrypt(key, iv, aad, C.c_size_t(len(aad)), plaintext, C.c_size_t(len(plaintext)), ct, tag)
    return ct.raw[:len(plaintext)] + tag.raw


def aes256_gcm_decrypt(key: bytes, iv: bytes, sealed: bytes, aad: bytes = b"") -> bytes:
    if len(key) != 32 or len(iv) != 12 or len(sealed) < 16:
        raise ValueError("key must be 32 bytes, iv 12 bytes and the input at least a tag long")
    ct, tag = sealed[:-16], sealed[-16:]
    pt = _buf(max(len(ct), 1))
    if _L().sx_aes256_gcm_decrypt(key, iv, aad, C.c_size_t(len(aad)), ct, C.c_size_t(len(ct)), tag, pt):
        raise ValueError("authentication failed")
    return pt.raw[:len(ct)]


def ed25519_public_key(seed: bytes) -> bytes:
    if len(seed) != 32:
        raise ValueError("seed must be 32 bytes")
    out = _buf(32)
    _L().sx_ed25519_public_key(seed, out)
    return out.raw


def ed25519_sign(seed: bytes, message: bytes) -> bytes:
    if len(seed) != 32:
        raise ValueError("seed must be 32 bytes")
    out = _buf(64)
    _L().sx_ed25519_sign(seed, message, C.c_size_t(len(message)), out)
    return out.raw


def ed25519_verify(public_key: bytes, message: bytes, signature: bytes) -> bool:
    if len(public_key) != 32 or len(signature) != 64:
        return False
    return bool(_L().sx_ed25519_verify(public_key, message, C.c_size_t(len(message)), signature))


def schnorr_public(secret: bytes) -> bytes:
    """P = x B on the Ed25519 group for a 32-byte secret (reduced modulo the group order)."""
    out = _buf(32)
    _L().sx_schnorr_public(secret, out)
    return out.raw


def schnorr_prove(secret: bytes, context: bytes = b"") -> bytes:
    """64-byte non-interactive proof of knowledge of `secret` for ``schnorr_public(secret)``, bound to `context`."""
    if len(secret) != 32:
        raise ValueError("secret must be 32 bytes")
    out = _buf(64)
    _L().sx_schnorr_prove(secret, context, C.c_size_t(len(context)), out)
    return out.raw


def schnorr_verify(public: bytes, proof: bytes, context: bytes = b"") -> bool:
    if len(public) != 32 or len(proof) != 64:
        return False
    return bool(_L().sx_schnorr_verify(public, context, C.c_size_t(len(context)), proof))


def argon2id(password: bytes, salt: bytes, time_cost: int = 3, memory_kib: int = 65536, lanes: int = 4, length: int = 32,
             secret: bytes = b"", ad: bytes = b"") -> bytes:
    """Argon2id (RFC 9106, version 0x13): memory-hard password hash / key derivation."""
    out = _buf(length)
    rc = _L().sx_argon2id(password, C.c_size_t(len(password)), salt, C.c_size_t(len(salt)), secret, C.c_size_t(len(secret)),
                          ad, C.c_size_t(len(ad)), C.c_uint32(time_cost), C.c_uint32(memory_kib), C.c_uint32(lanes), out,
                          C.c_uint32(length))
    if rc:
        raise ValueError("argon2id: need lanes >= 1, time_cost >= 1, length >= 4, memory_kib >= 8 * lanes, salt of 8+ bytes")
    return out.raw


def poly1305(key: bytes, message: bytes) -> bytes:
    """One-time authenticator (RFC 8439 section 2.5): 16-byte tag under a 32-byte one-time key."""
    if len(key) != 32:
        raise ValueError("key must be 32 bytes")
    out = _buf(16)
    _L().sx_poly1305(key, message, C.c_size_t(len(message)), out)
    return out.raw


def blake3(data: bytes, length: int = 32, key: bytes = None) -> bytes:
    """BLAKE3 hash (or keyed hash with a 32-byte key) with any output length."""
    if key is not None and len(key) != 32:
        raise ValueError("key must be 32 bytes")
    out = _buf(length)
    _L().sx_blake3(data, C.c_size_t(len(data)), key, out, C.c_size_t(length))
    return out.raw


def shake128(data: bytes, length: int) -> bytes:
    out = _buf(length)
    _L().sx_shake128(data, C.c_size_t(len(data)), out, C.c_size_t(length))
    return out.raw


# ------------------------------------------------------------------------------------------ post-quantum
_MLKEM_K = {512: 2, 768: 3, 1024: 4}


def mlkem_sizes(level: int = 768):
    """(encapsulation key, decapsulation key, ciphertext) lengths in bytes for ML-KEM-512 / 768 / 1024."""
    ek, dk, ct = C.c_int(), C.c_int(), C.c_int()
    if level not in _MLKEM_K or _L().sx_mlkem_sizes(_MLKEM_K[level], C.byref(ek), C.byref(dk), C.byref(ct)) != 0:
        raise ValueError("level must be 512, 768 or 1024")
    return ek.value, dk.value, ct.value


def mlkem_keygen(level: int = 768, seed: bytes = None):
    """ML-KEM (FIPS 203) key pair -> (encapsulation key, decapsulation key). `seed` is the 64-byte d || z of the
    standard's internal key generation (fresh randomness when omitted)."""
    import os
    seed = os.urandom(64) if seed is None else seed
    if len(seed) != 64:
        raise ValueError("seed must be 64 bytes (d || z)")
    n_ek, n_dk, _ = mlkem_sizes(level)
    ek, dk = _buf(n_ek), _buf(n_dk)
    _L().sx_mlkem_keygen(_MLKEM_K[level], seed[:32], seed[32:], ek, dk)
    return ek.raw, dk.raw


def mlkem_encaps(ek: bytes, level: int = 768, message: bytes = None):
    """-> (shared secret of 32 bytes, ciphertext). `message` is the 32-byte randomness of the standard's internal
    encapsulation (fresh when omitted). Raises on a key of the wrong length or with out-of-range coefficients."""
    import os
    n_ek, _, n_ct = mlkem_sizes(level)
    if len(ek) != n_ek:
        raise ValueError(f"encapsulation key must be {n_ek} bytes")
    message = os.urandom(32) if message is None else message
    if len(message) != 32:
        raise ValueError("message must be 32 bytes")
    ct, ss = _buf(n_ct), _buf(32)
    if _L().sx_mlkem_encaps(_MLKEM_K[level], ek, message, ct, ss) != 0:
        raise ValueError("encapsulation key fails the modulus check")
    return ss.raw, ct.raw


def mlkem_decaps(dk: bytes, ct: bytes, level: int = 768) -> bytes:
    """Shared secret for a ciphertext. A forged or damaged ciphertext gives an unrelated pseudo-random secret
    (implicit rejection), not an error."""
    _, n_dk, n_ct = mlkem_sizes(level)
    if len(dk) != n_dk or len(ct) != n_ct:
        raise ValueError(f"decapsulation key must be {n_dk} bytes and the ciphertext {n_ct} bytes")
    ss = _buf(32)
    _L().sx_mlkem_decaps(_MLKEM_K[level], dk, ct, ss)
    return ss.raw


_MLDSA_LEVELS = (44, 65, 87)


def mldsa_sizes(level: int = 65):
    """(public key, private key, signature) lengths in bytes for ML-DSA-44 / 65 / 87."""
    pk, sk, sig = C.c_int(), C.c_int(), C.c_int()
    if level not in _MLDSA_LEVELS or _L().sx_mldsa_sizes(level, C.byref(pk), C.byref(sk), C.byref(sig)) != 0:
        raise ValueError("level must be 44, 65 or 87")
    return pk.value, sk.value, sig.value


def mldsa_keygen(level: int = 65, seed: bytes = None):
    """ML-DSA (FIPS 204) key pair from a 32-byte seed -> (public key, private key)."""
    import os
    seed = os.urandom(32) if seed is None else seed
    if len(seed) != 32:
        raise ValueError("seed must be 32 bytes")
    n_pk, n_sk, _ = mldsa_sizes(level)
    pk, sk = _buf(n_pk), _buf(n_sk)
    _L().sx_mldsa_keygen(level, seed, pk, sk)
    return pk.raw, sk.raw


def mldsa_sign(sk: bytes, message: bytes, level: int = 65, context: bytes = b"", deterministic: bool = False) -> bytes:
    """Signature of `message` (pure ML-DSA with a context string of at most 255 bytes). Hedged with 32 fresh random
    bytes unless `deterministic`."""
    import os
    _, n_sk, n_sig = mldsa_sizes(level)
    if len(sk) != n_sk or len(context) > 255:
        raise ValueError(f"private key must be {n_sk} bytes and the context at most 255 bytes")
    rnd = bytes(32) if deterministic else os.urandom(32)
    sig = _buf(n_sig)
    if _L().sx_mldsa_sign(level, sk, message, C.c_size_t(len(message)), context, C.c_size_t(len(context)), rnd, sig) != 0:
        raise RuntimeError("ML-DSA signing failed")
    return sig.raw


def mldsa_verify(pk: bytes, message: bytes, signature: bytes, level: int = 65, context: bytes = b"") -> bool:
    n_pk, _, n_sig = mldsa_sizes(level)
    if len(pk) != n_pk or len(signature) != n_sig or len(context) > 255:
        return False
    return _L().sx_mldsa_verify(level, pk, message, C.c_size_t(len(message)), context, C.c_size_t(len(context)), signature) == 1


_SLH_VARIANTS = {"128f": 0, "128s": 1}


def slhdsa_sizes(variant: str = "128f"):
    """(public key, private key, signature) lengths for SLH-DSA-SHAKE-128f / 128s."""
    pk, sk, sig = C.c_int(), C.c_int(), C.c_int()
    if variant not in _SLH_VARIANTS or _L().sx_slhdsa_sizes(_SLH_VARIANTS[variant], C.byref(pk), C.byref(sk), C.byref(sig)) != 0:
        raise ValueError("variant must be '128f' or '128s'")
    return pk.value, sk.value, sig.value


def slhdsa_keygen(variant: str = "128f", seed: bytes = None):
    """SLH-DSA (FIPS 205, SHAKE) key pair from the 48-byte SK.seed || SK.prf || PK.seed -> (public key, private key)."""
    import os
    seed = os.urandom(48) if seed is None else seed
    if len(seed) != 48:
        raise ValueError("seed must be 48 bytes")
    n_pk, n_sk, _ = slhdsa_sizes(variant)
    pk, sk = _buf(n_pk), _buf(n_sk)
    _L().sx_slhdsa_keygen(_SLH_VARIANTS[variant], seed, pk, sk)
    return pk.raw, sk.raw


def slhdsa_sign(sk: bytes, message: bytes, variant: str = "128f", context: bytes = b"", deterministic: bool = False) -> bytes:
    import os
    _, n_sk, n_sig = slhdsa_sizes(variant)
    if len(sk) != n_sk or len(context) > 255:
        raise ValueError(f"private key must be {n_sk} bytes and the context at most 255 bytes")
    sig = _buf(n_sig)
    rnd = None if deterministic else os.urandom(16)
    if _L().sx_slhdsa_sign(_SLH_VARIANTS[variant], sk, message, C.c_size_t(len(message)), context, C.c_size_t(len(context)), rnd, sig) != 0:
        raise RuntimeError("SLH-DSA signing failed")
    return sig.raw


def slhdsa_verify(pk: bytes, message: bytes, signature: bytes, variant: str = "128f", context: bytes = b"") -> bool:
    n_pk, _, n_sig = slhdsa_sizes(variant)
    if len(pk) != n_pk or len(signature) != n_sig or len(context) > 255:
        return False
    return _L().sx_slhdsa_verify(_SLH_VARIANTS[variant], pk, message, C.c_size_t(len(message)), context,
                                 C.c_size_t(len(context)), signature) == 1


class KyberKEM:
    """ML-KEM behind the reference's class shape (``crypto_kem.py:17-54``): ``keypair() -> (pk, sk)``,
    ``encapsulate(pk) -> (ciphertext, shared secret)``, ``decapsulate(sk, ciphertext) -> shared secret``."""
    MODE_ML_KEM_512, MODE_ML_KEM_768, MODE_ML_KEM_1024 = 512, 768, 1024

    def __init__(self, mode: int = 1024):
        self.mode = mode

    def keypair(self, seed: bytes = None):
        return mlkem_keygen(self.mode, None if seed is None else sha3_512(seed))

    def encapsulate(self, pk: bytes):
        ss, ct = mlkem_encaps(pk, self.mode)
        return ct, ss

    def decapsulate(self, sk: bytes, ct: bytes):
        return mlkem_decaps(sk, ct, self.mode)


class Dilithium:
    """ML-DSA behind the reference's class shape (``crypto_sign.py:93-131``); modes 2 / 3 / 5 are ML-DSA-44 / 65 / 87."""
    MODE_ML_DSA_44, MODE_ML_DSA_65, MODE_ML_DSA_87 = 2, 3, 5
    _LEVEL = {2: 44, 3: 65, 5: 87}

    def __init__(self, mode: int = 2):
        self.mode, self.level = mode, self._LEVEL[mode]

    def keypair(self, seed: bytes = None):
        return mldsa_keygen(self.level, None if seed is None else sha3_256(seed))

    def sign(self, sk: bytes, msg: bytes) -> bytes:
        return mldsa_sign(sk, msg, self.level)

    def verify(self, pk: bytes, msg: bytes, sig: bytes) -> bool:
        return mldsa_verify(pk, msg, sig, self.level)


class SphincsPlus:
    """SLH-DSA-SHAKE behind the reference's class shape (``crypto_sign.py:136-168``); variants "128f" and "128s"."""

    def __init__(self, variant: str = "128f"):
        self.variant = variant

    def keypair(self, seed: bytes = None):
        return slhdsa_keygen(self.variant, None if seed is None else shake256(seed, 48))

    def sign(self, sk: bytes, msg: bytes) -> bytes:
        return slhdsa_sign(sk, msg, self.variant)

    def verify(self, pk: bytes, msg: bytes, sig: bytes) -> bool:
        return slhdsa_verify(pk, msg, sig, self.variant)


class MontgomeryMul:
    """Montgomery modular multiplication for an odd modulus (the reference's ``MontgomeryMul``, ``crypto_asm.py:147``,
    is ``a * b * inv % mod``). ``to_mont`` / ``from_mont`` convert, ``mont_mul`` multiplies two Montgomery-form values
    with one reduction (no division by the modulus), ``pow`` is square-and-multiply in that form."""

    def __init__(self, modulus: int = None):
        if modulus is not None:
            if modulus % 2 == 0 or modulus < 3:
                raise ValueError("modulus must be odd and >= 3")
            self.n = modulus
            self.bits = modulus.bit_length()
            self.r_mask = (1 << self.bits) - 1
            self.n_prime = (-pow(modulus, -1, 1 << self.bits)) & self.r_mask
            self.r2 = pow(1 << self.bits, 2, modulus)

    def _redc(self, t: int) -> int:
        m = ((t & self.r_mask) * self.n_prime) & self.r_mask
        u = (t + m * self.n) >> self.bits
        return u - self.n if u >= self.n else u

    def to_mont(self, a: int) -> int:
        return self._redc((a % self.n) * self.r2)

    def from_mont(self, a: int) -> int:
        return self._redc(a)

    def mont_mul(self, a: int, b: int) -> int:
        return self._redc(a * b)

    def pow(self, base: int, exponent: int) -> int:
        x, acc = self.to_mont(base), self.to_mont(1)
        while exponent:
            if exponent & 1:
                acc = self.mont_mul(acc, x)
            x = self.mont_mul(x, x)
            exponent >>= 1
        return self.from_mont(acc)

    def mul(self, a: int, b: int, mod: int, inv: int = 1) -> int:
        return (a * b * inv) % mod
