// S0 crypto primitives in portable C++ (the reference implements them in C plus x86-64 MASM under security/crypto):
// SHA-256, HMAC-SHA256, HKDF, PBKDF2, ChaCha20, Poly1305, ChaCha20-Poly1305 AEAD (RFC 8439), SipHash-2-4, X25519
// (RFC 7748), HMAC-DRBG, constant-time comparison, and an S1 guarded allocator with canaries.
// Host-side and off the hot path; validated against RFC / NIST test vectors in tests/test_security_cpu.py.
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace {

// ---------------------------------------------------------------- SHA-256
const uint32_t K256[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5, 0xd807aa98, 0x12835b01,
    0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174, 0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc,
    0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da, 0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147,
    0x06ca6351, 0x14292967, 0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070, 0x19a4c116, 0x1e376c08,
    0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3, 0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208,
    0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
struct Sha256 {
  uint32_t h[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a, 0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  uint8_t buf[64];
  uint64_t len = 0;
  size_t fill = 0;
  void block(const uint8_t* p) {
    uint32_t w[64];
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
    for (int i = 16; i < 64; ++i) {
      const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
      const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 64; ++i) {
      const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K256[i] + w[i];
      const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  void update(const uint8_t* p, size_t n) {
    len += n;
    while (n) {
      const size_t k = n < 64 - fill ? n : 64 - fill;
      memcpy(buf + fill, p, k);
      fill += k; p += k; n -= k;
      if (fill == 64) { block(buf); fill = 0; }
    }
  }
  void final(uint8_t out[32]) {
    const uint64_t bits = len * 8;
    uint8_t pad = 0x80;
    update(&pad, 1);
    pad = 0;
    while (fill != 56) update(&pad, 1);
    uint8_t lb[8];
    for (int i = 0; i < 8; ++i) lb[i] = (uint8_t)(bits >> (56 - 8 * i));
    update(lb, 8);
    for (int i = 0; i < 8; ++i) { out[4 * i] = h[i] >> 24; out[4 * i + 1] = h[i] >> 16; out[4 * i + 2] = h[i] >> 8; out[4 * i + 3] = h[i]; }
  }
};
void sha256(const uint8_t* p, size_t n, uint8_t out[32]) {
  Sha256 s;
  s.update(p, n);
  s.final(out);
}
void hmac_sha256(const uint8_t* key, size_t kn, const uint8_t* msg, size_t mn, uint8_t out[32]) {
  uint8_t k[64] = {0}, ipad[64], opad[64], inner[32];
  if (kn > 64) sha256(key, kn, k); else memcpy(k, key, kn);
  for (int i = 0; i < 64; ++i) { ipad[i] = k[i] ^ 0x36; opad[i] = k[i] ^ 0x5c; }
  Sha256 a;
  a.update(ipad, 64); a.update(msg, mn); a.final(inner);
  Sha256 b;
  b.update(opad, 64); b.update(inner, 32); b.final(out);
}

// ---------------------------------------------------------------- ChaCha20 / Poly1305
inline uint32_t rotl(uint32_t x, int n) { return (x << n) | (x >> (32 - n)); }
inline uint32_t ld32(const uint8_t* p) { return (uint32_t)p[0] | (uint32_t)p[1] << 8 | (uint32_t)p[2] << 16 | (uint32_t)p[3] << 24; }
inline void st32(uint8_t* p, uint32_t v) { p[0] = v; p[1] = v >> 8; p[2] = v >> 16; p[3] = v >> 24; }
void chacha_block(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], uint8_t out[64]) {
  uint32_t s[16] = {0x61707865, 0x3320646e, 0x79622d32, 0x6b206574};
  for (int i = 0; i < 8; ++i) s[4 + i] = ld32(key + 4 * i);
  s[12] = counter;
  for (int i = 0; i < 3; ++i) s[13 + i] = ld32(nonce + 4 * i);
  uint32_t x[16];
  memcpy(x, s, sizeof(s));
#define QR(a, b, c, d) x[a] += x[b]; x[d] = rotl(x[d] ^ x[a], 16); x[c] += x[d]; x[b] = rotl(x[b] ^ x[c], 12); \
                       x[a] += x[b]; x[d] = rotl(x[d] ^ x[a], 8); x[c] += x[d]; x[b] = rotl(x[b] ^ x[c], 7);
  for (int i = 0; i < 10; ++i) {
    QR(0, 4, 8, 12) QR(1, 5, 9, 13) QR(2, 6, 10, 14) QR(3, 7, 11, 15)
    QR(0, 5, 10, 15) QR(1, 6, 11, 12) QR(2, 7, 8, 13) QR(3, 4, 9, 14)
  }
#undef QR
  for (int i = 0; i < 16; ++i) st32(out + 4 * i, x[i] + s[i]);
}
void chacha_xor(const uint8_t key[32], uint32_t counter, const uint8_t nonce[12], const uint8_t* in, uint8_t* out, size_t n) {
  uint8_t ks[64];
  for (size_t off = 0; off < n; off += 64) {
    chacha_block(key, counter++, nonce, ks);
    const size_t k = n - off < 64 ? n - off : 64;
    for (size_t i = 0; i < k; ++i) out[off + i] = in[off + i] ^ ks[i];
  }
}
// Poly1305 with 26-bit limbs
void poly1305(const uint8_t key[32], const uint8_t* m, size_t n, uint8_t tag[16]) {
  uint32_t r0 = ld32(key) & 0x3ffffff, r1 = (ld32(key + 3) >> 2) & 0x3ffff03, r2 = (ld32(key + 6) >> 4) & 0x3ffc0ff,
           r3 = (ld32(key + 9) >> 6) & 0x3f03fff, r4 = (ld32(key + 12) >> 8) & 0x00fffff;
  uint32_t s1 = r1 * 5, s2 = r2 * 5, s3 = r3 * 5, s4 = r4 * 5;
  uint32_t h0 = 0, h1 = 0, h2 = 0, h3 = 0, h4 = 0;
  while (n) {
    uint8_t blk[17] = {0};
    const size_t k = n < 16 ? n : 16;
    memcpy(blk, m, k);
    blk[k] = 1;
    h0 += ld32(blk) & 0x3ffffff;
    h1 += (ld32(blk + 3) >> 2) & 0x3ffffff;
    h2 += (ld32(blk + 6) >> 4) & 0x3ffffff;
    h3 += (ld32(blk + 9) >> 6) & 0x3ffffff;
    h4 += (ld32(blk + 12) >> 8) | ((uint32_t)blk[16] << 24);
    const uint64_t d0 = (uint64_t)h0 * r0 + (uint64_t)h1 * s4 + (uint64_t)h2 * s3 + (uint64_t)h3 * s2 + (uint64_t)h4 * s1;
    uint64_t d1 = (uint64_t)h0 * r1 + (uint64_t)h1 * r0 + (uint64_t)h2 * s4 + (uint64_t)h3 * s3 + (uint64_t)h4 * s2;
    uint64_t d2 = (uint64_t)h0 * r2 + (uint64_t)h1 * r1 + (uint64_t)h2 * r0 + (uint64_t)h3 * s4 + (uint64_t)h4 * s3;
    uint64_t d3 = (uint64_t)h0 * r3 + (uint64_t)h1 * r2 + (uint64_t)h2 * r1 + (uint64_t)h3 * r0 + (uint64_t)h4 * s4;
    uint64_t d4 = (uint64_t)h0 * r4 + (uint64_t)h1 * r3 + (uint64_t)h2 * r2 + (uint64_t)h3 * r1 + (uint64_t)h4 * r0;
    uint32_t c = (uint32_t)(d0 >> 26); h0 = (uint32_t)d0 & 0x3ffffff;
    d1 += c; c = (uint32_t)(d1 >> 26); h1 = (uint32_t)d1 & 0x3ffffff;
    d2 += c; c = (uint32_t)(d2 >> 26); h2 = (uint32_t)d2 & 0x3ffffff;
    d3 += c; c = (uint32_t)(d3 >> 26); h3 = (uint32_t)d3 & 0x3ffffff;
    d4 += c; c = (uint32_t)(d4 >> 26); h4 = (uint32_t)d4 & 0x3ffffff;
    h0 += c * 5; c = h0 >> 26; h0 &= 0x3ffffff; h1 += c;
    m += k; n -= k;
  }
  uint32_t c = h1 >> 26; h1 &= 0x3ffffff; h2 += c; c = h2 >> 26; h2 &= 0x3ffffff; h3 += c; c = h3 >> 26; h3 &= 0x3ffffff;
  h4 += c; c = h4 >> 26; h4 &= 0x3ffffff; h0 += c * 5; c = h0 >> 26; h0 &= 0x3ffffff; h1 += c;
  uint32_t g0 = h0 + 5; c = g0 >> 26; g0 &= 0x3ffffff;
  uint32_t g1 = h1 + c; c = g1 >> 26; g1 &= 0x3ffffff;
  uint32_t g2 = h2 + c; c = g2 >> 26; g2 &= 0x3ffffff;
  uint32_t g3 = h3 + c; c = g3 >> 26; g3 &= 0x3ffffff;
  uint32_t g4 = h4 + c - (1u << 26);
  const uint32_t mask = (g4 >> 31) - 1;  // all ones when h >= p
  h0 = (h0 & ~mask) | (g0 & mask); h1 = (h1 & ~mask) | (g1 & mask); h2 = (h2 & ~mask) | (g2 & mask);
  h3 = (h3 & ~mask) | (g3 & mask); h4 = (h4 & ~mask) | (g4 & mask);
  uint64_t f0 = ((h0) | (h1 << 26)) & 0xffffffff, f1 = ((h1 >> 6) | (h2 << 20)) & 0xffffffff,
           f2 = ((h2 >> 12) | (h3 << 14)) & 0xffffffff, f3 = ((h3 >> 18) | (h4 << 8)) & 0xffffffff;
  f0 += ld32(key + 16); f1 += ld32(key + 20) + (f0 >> 32); f2 += ld32(key + 24) + (f1 >> 32); f3 += ld32(key + 28) + (f2 >> 32);
  st32(tag, (uint32_t)f0); st32(tag + 4, (uint32_t)f1); st32(tag + 8, (uint32_t)f2); st32(tag + 12, (uint32_t)f3);
}
void aead_tag(const uint8_t key[32], const uint8_t nonce[12], const uint8_t* aad, size_t an, const uint8_t* ct, size_t cn, uint8_t tag[16]) {
  uint8_t otk[64];
  chacha_block(key, 0, nonce, otk);
  std::vector<uint8_t> mac;
  mac.insert(mac.end(), aad, aad + an);
  mac.resize((mac.size() + 15) / 16 * 16, 0);
  mac.insert(mac.end(), ct, ct + cn);
  mac.resize((mac.size() + 15) / 16 * 16, 0);
  for (int i = 0; i < 8; ++i) mac.push_back((uint8_t)((uint64_t)an >> (8 * i)));
  for (int i = 0; i < 8; ++i) mac.push_back((uint8_t)((uint64_t)cn >> (8 * i)));
  poly1305(otk, mac.data(), mac.size(), tag);
}

// ---------------------------------------------------------------- X25519 (field arithmetic with 16 x 16-bit limbs)
typedef int64_t gf[16];
void car(gf o) {
  for (int i = 0; i < 16; ++i) {
    o[i] += (1LL << 16);
    const int64_t c = o[i] >> 16;
    o[(i + 1) * (i < 15)] += c - 1 + 37 * (c - 1) * (i == 15);
    o[i] -= c * 65536;  // not c << 16: shifting a negative value is undefined before C++20
  }
}
void sel(gf p, gf q, int b) {
  const int64_t c = ~(b - 1);
  for (int i = 0; i < 16; ++i) { const int64_t t = c & (p[i] ^ q[i]); p[i] ^= t; q[i] ^= t; }
}
void pack(uint8_t* o, const gf n) {
  gf m, t;
  memcpy(t, n, sizeof(gf));
  car(t); car(t); car(t);
  for (int j = 0; j < 2; ++j) {
    m[0] = t[0] - 0xffed;
    for (int i = 1; i < 15; ++i) { m[i] = t[i] - 0xffff - ((m[i - 1] >> 16) & 1); m[i - 1] &= 0xffff; }
    m[15] = t[15] - 0x7fff - ((m[14] >> 16) & 1);
    const int b = (m[15] >> 16) & 1;
    m[14] &= 0xffff;
    sel(t, m, 1 - b);
  }
  for (int i = 0; i < 16; ++i) { o[2 * i] = t[i] & 0xff; o[2 * i + 1] = t[i] >> 8; }
}
void unpack(gf o, const uint8_t* n) {
  for (int i = 0; i < 16; ++i) o[i] = n[2 * i] + ((int64_t)n[2 * i + 1] << 8);
  o[15] &= 0x7fff;
}
void A(gf o, const gf a, const gf b) { for (int i = 0; i < 16; ++i) o[i] = a[i] + b[i]; }
void Z(gf o, const gf a, const gf b) { for (int i = 0; i < 16; ++i) o[i] = a[i] - b[i]; }
void M(gf o, const gf a, const gf b) {
  int64_t t[31] = {0};
  for (int i = 0; i < 16; ++i) for (int j = 0; j < 16; ++j) t[i + j] += a[i] * b[j];
  for (int i = 0; i < 15; ++i) t[i] += 38 * t[i + 16];
  for (int i = 0; i < 16; ++i) o[i] = t[i];
  car(o); car(o);
}
void inv(gf o, const gf i) {
  gf c;
  memcpy(c, i, sizeof(gf));
  for (int a = 253; a >= 0; --a) { M(c, c, c); if (a != 2 && a != 4) M(c, c, i); }
  memcpy(o, c, sizeof(gf));
}
const gf k121665 = {0xDB41, 1};
void x25519(uint8_t* q, const uint8_t* n, const uint8_t* p) {
  uint8_t z[32];
  gf x, a, b, c, d, e, f;
  memcpy(z, n, 32);
  z[31] = (n[31] & 127) | 64;
  z[0] &= 248;
  unpack(x, p);
  for (int i = 0; i < 16; ++i) { b[i] = x[i]; d[i] = a[i] = c[i] = 0; }
  a[0] = d[0] = 1;
  for (int i = 254; i >= 0; --i) {
    const int r = (z[i >> 3] >> (i & 7)) & 1;
    sel(a, b, r); sel(c, d, r);
    A(e, a, c); Z(a, a, c); A(c, b, d); Z(b, b, d); M(d, e, e); M(f, a, a); M(a, c, a); M(c, b, e);
    A(e, a, c); Z(a, a, c); M(b, a, a); Z(c, d, f); M(a, c, k121665); A(a, a, d); M(c, c, a); M(a, d, f);
    M(d, b, x); M(b, e, e);
    sel(a, b, r); sel(c, d, r);
  }
  inv(c, c);
  M(a, a, c);
  pack(q, a);
}

}  // namespace

extern "C" {
void sx_sha256(const uint8_t* p, size_t n, uint8_t* out32) { sha256(p, n, out32); }
void sx_hmac_sha256(const uint8_t* k, size_t kn, const uint8_t* m, size_t mn, uint8_t* out32) { hmac_sha256(k, kn, m, mn, out32); }
void sx_hkdf_sha256(const uint8_t* ikm, size_t in, const uint8_t* salt, size_t sn, const uint8_t* info, size_t fn, uint8_t* out, size_t on) {
  uint8_t prk[32], zero[32] = {0}, t[32];
  hmac_sha256(sn ? salt : zero, sn ? sn : 32, ikm, in, prk);
  size_t done = 0, tl = 0;
  for (uint8_t ctr = 1; done < on; ++ctr) {
    std::vector<uint8_t> msg(t, t + tl);
    msg.insert(msg.end(), info, info + fn);
    msg.push_back(ctr);
    hmac_sha256(prk, 32, msg.data(), msg.size(), t);
    tl = 32;
    const size_t k = on - done < 32 ? on - done : 32;
    memcpy(out + done, t, k);
    done += k;
  }
}
void sx_pbkdf2_sha256(const uint8_t* pw, size_t pn, const uint8_t* salt, size_t sn, int iters, uint8_t* out, size_t on) {
  for (uint32_t blk = 1, done = 0; done < on; ++blk) {
    std::vector<uint8_t> s(salt, salt + sn);
    for (int i = 3; i >= 0; --i) s.push_back((uint8_t)(blk >> (8 * i)));
    uint8_t u[32], t[32];
    hmac_sha256(pw, pn, s.data(), s.size(), u);
    memcpy(t, u, 32);
    for (int i = 1; i < iters; ++i) {
      hmac_sha256(pw, pn, u, 32, u);
      for (int j = 0; j < 32; ++j) t[j] ^= u[j];
    }
    const size_t k = on - done < 32 ? on - done : 32;
    memcpy(out + done, t, k);
    done += (uint32_t)k;
  }
}
void sx_chacha20(const uint8_t* key32, uint32_t counter, const uint8_t* nonce12, const uint8_t* in, uint8_t* out, size_t n) {
  chacha_xor(key32, counter, nonce12, in, out, n);
}
void sx_poly1305(const uint8_t* key32, const uint8_t* m, size_t n, uint8_t* tag16) { poly1305(key32, m, n, tag16); }
void sx_aead_encrypt(const uint8_t* key32, const uint8_t* nonce12, const uint8_t* aad, size_t an, const uint8_t* pt, size_t n,
                     uint8_t* ct, uint8_t* tag16) {
  chacha_xor(key32, 1, nonce12, pt, ct, n);
  aead_tag(key32, nonce12, aad, an, ct, n, tag16);
}
int sx_ct_equal(const uint8_t* a, const uint8_t* b, size_t n) {
  uint8_t d = 0;
  for (size_t i = 0; i < n; ++i) d |= a[i] ^ b[i];
  return d == 0;
}
// returns 0 and writes the plaintext only when the tag verifies
int sx_aead_decrypt(const uint8_t* key32, const uint8_t* nonce12, const uint8_t* aad, size_t an, const uint8_t* ct, size_t n,
                    const uint8_t* tag16, uint8_t* pt) {
  uint8_t tag[16];
  aead_tag(key32, nonce12, aad, an, ct, n, tag);
  if (!sx_ct_equal(tag, tag16, 16)) return -1;
  chacha_xor(key32, 1, nonce12, ct, pt, n);
  return 0;
}
uint64_t sx_siphash24(const uint8_t* key16, const uint8_t* m, size_t n) {
  auto rl = [](uint64_t x, int b) { return (x << b) | (x >> (64 - b)); };
  uint64_t k0, k1;
  memcpy(&k0, key16, 8); memcpy(&k1, key16 + 8, 8);
  uint64_t v0 = k0 ^ 0x736f6d6570736575ull, v1 = k1 ^ 0x646f72616e646f6dull, v2 = k0 ^ 0x6c7967656e657261ull, v3 = k1 ^ 0x7465646279746573ull;
  auto round = [&] {
    v0 += v1; v1 = rl(v1, 13); v1 ^= v0; v0 = rl(v0, 32); v2 += v3; v3 = rl(v3, 16); v3 ^= v2;
    v0 += v3; v3 = rl(v3, 21); v3 ^= v0; v2 += v1; v1 = rl(v1, 17); v1 ^= v2; v2 = rl(v2, 32);
  };
  const size_t full = n / 8 * 8;
  for (size_t i = 0; i < full; i += 8) {
    uint64_t w;
    memcpy(&w, m + i, 8);
    v3 ^= w; round(); round(); v0 ^= w;
  }
  uint64_t b = (uint64_t)n << 56;
  for (size_t i = full; i < n; ++i) b |= (uint64_t)m[i] << (8 * (i - full));
  v3 ^= b; round(); round(); v0 ^= b;
  v2 ^= 0xff; round(); round(); round(); round();
  return v0 ^ v1 ^ v2 ^ v3;
}
void sx_x25519(uint8_t* out32, const uint8_t* scalar32, const uint8_t* point32) { x25519(out32, scalar32, point32); }
void sx_x25519_base(uint8_t* out32, const uint8_t* scalar32) {
  uint8_t base[32] = {9};
  x25519(out32, scalar32, base);
}
// HMAC-DRBG (SP 800-90A) state = K || V (64 bytes)
void sx_drbg_init(uint8_t* state64, const uint8_t* seed, size_t n) {
  memset(state64, 0, 32);
  memset(state64 + 32, 1, 32);
  for (uint8_t sep = 0; sep < 2; ++sep) {
    std::vector<uint8_t> m(state64 + 32, state64 + 64);
    m.push_back(sep);
    m.insert(m.end(), seed, seed + n);
    hmac_sha256(state64, 32, m.data(), m.size(), state64);
    hmac_sha256(state64, 32, state64 + 32, 32, state64 + 32);
  }
}
void sx_drbg_generate(uint8_t* state64, uint8_t* out, size_t n) {
  size_t done = 0;
  while (done < n) {
    hmac_sha256(state64, 32, state64 + 32, 32, state64 + 32);
    const size_t k = n - done < 32 ? n - done : 32;
    memcpy(out + done, state64 + 32, k);
    done += k;
  }
  std::vector<uint8_t> m(state64 + 32, state64 + 64);
  m.push_back(0);
  hmac_sha256(state64, 32, m.data(), m.size(), state64);
  hmac_sha256(state64, 32, state64 + 32, 32, state64 + 32);
}
// S1 guarded allocation: [canary 16][size 8][pad 8][user bytes][canary 16]; free checks both canaries and wipes.
static const uint8_t kCanary[16] = {0xDE, 0xAD, 0xBE, 0xEF, 0x5A, 0xA5, 0xC3, 0x3C, 0x96, 0x69, 0x0F, 0xF0, 0x11, 0xEE, 0x77, 0x88};
void* sx_guarded_alloc(size_t n) {
  uint8_t* raw = (uint8_t*)malloc(n + 48);
  if (!raw) return nullptr;
  memcpy(raw, kCanary, 16);
  memcpy(raw + 16, &n, sizeof(size_t));
  memcpy(raw + 32 + n, kCanary, 16);
  memset(raw + 32, 0, n);
  return raw + 32;
}
// 0 ok, 1 front canary smashed, 2 rear canary smashed
int sx_guarded_check(const void* p) {
  const uint8_t* raw = (const uint8_t*)p - 32;
  size_t n;
  memcpy(&n, raw + 16, sizeof(size_t));
  if (memcmp(raw, kCanary, 16)) return 1;
  if (memcmp(raw + 32 + n, kCanary, 16)) return 2;
  return 0;
}
int sx_guarded_free(void* p) {
  const int rc = sx_guarded_check(p);
  uint8_t* raw = (uint8_t*)p - 32;
  size_t n;
  memcpy(&n, raw + 16, sizeof(size_t));
  volatile uint8_t* v = (volatile uint8_t*)p;
  for (size_t i = 0; i < n; ++i) v[i] = 0;
  free(raw);
  return rc;
}
}
