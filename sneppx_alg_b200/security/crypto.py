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
