// Post-quantum key encapsulation: ML-KEM (FIPS 203, the standardised form of Kyber) at parameter sets 512 / 768 / 1024.
//
// Reference counterpart: security/crypto/post_quantum (Kyber). Written from FIPS 203: the number-theoretic transform
// over Z_3329 with zeta = 17, centred-binomial sampling from SHAKE-256, rejection sampling of the public matrix from
// SHAKE-128, coefficient compression, and the Fujisaki-Okamoto transform with implicit rejection. The tests check key
// generation from a seed, encapsulation and decapsulation in both directions against an independent implementation.
// Arithmetic uses plain integer division and is not hardened against timing side channels.
#include <cstdint>
#include <cstring>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" {
void sx_sha3_256(const void* msg, size_t len, void* out32);
void sx_sha3_512(const void* msg, size_t len, void* out64);
void sx_shake256(const void* msg, size_t len, void* out, size_t outlen);
void sx_shake128(const void* msg, size_t len, void* out, size_t outlen);
}

namespace {

constexpr int N = 256, Q = 3329;
typedef int16_t poly[N];

struct Params { int k, eta1, eta2, du, dv; };
bool params_for(int k, Params& p) {
  if (k == 2) p = {2, 3, 2, 10, 4};
  else if (k == 3) p = {3, 2, 2, 10, 4};
  else if (k == 4) p = {4, 2, 2, 11, 5};
  else return false;
  return true;
}

int zetas[128], gammas[128];
bool tables_ready = false;
int powmod(int b, int e) { long r = 1, x = b; while (e) { if (e & 1) r = r * x % Q; x = x * x % Q; e >>= 1; } return (int)r; }
int bitrev7(int i) { int r = 0; for (int b = 0; b < 7; ++b) r |= ((i >> b) & 1) << (6 - b); return r; }
void init_tables() {
  if (tables_ready) return;
  for (int i = 0; i < 128; ++i) { zetas[i] = powmod(17, bitrev7(i)); gammas[i] = powmod(17, 2 * bitrev7(i) + 1); }
  tables_ready = true;
}
inline int16_t modq(int x) { int r = x % Q; return (int16_t)(r < 0 ? r + Q : r); }

void ntt(poly f) {
  int k = 1;
  for (int len = 128; len >= 2; len >>= 1)
    for (int start = 0; start < N; start += 2 * len) {
      const int z = zetas[k++];
      for (int j = start; j < start + len; ++j) {
        const int t = z * f[j + len] % Q;
        f[j + len] = modq(f[j] - t);
        f[j] = modq(f[j] + t);
      }
    }
}
void intt(poly f) {
  int k = 127;
  for (int len = 2; len <= 128; len <<= 1)
    for (int start = 0; start < N; start += 2 * len) {
      const int z = zetas[k--];
      for (int j = start; j < start + len; ++j) {
        const int t = f[j];
        f[j] = modq(t + f[j + len]);
        f[j + len] = modq(z * (f[j + len] - t));
      }
    }
  for (int i = 0; i < N; ++i) f[i] = modq(f[i] * 3303);   // 128^-1 mod q
}
// acc += a * b in the NTT domain (128 products of degree-1 polynomials modulo X^2 - gamma_i)
void mul_acc(poly acc, const poly a, const poly b) {
  for (int i = 0; i < 128; ++i) {
    const int a0 = a[2 * i], a1 = a[2 * i + 1], b0 = b[2 * i], b1 = b[2 * i + 1];
    const int c0 = (a0 * b0 + (a1 * b1 % Q) * gammas[i]) % Q;
    const int c1 = (a0 * b1 + a1 * b0) % Q;
    acc[2 * i] = modq(acc[2 * i] + c0);
    acc[2 * i + 1] = modq(acc[2 * i + 1] + c1);
  }
}

void byte_encode(const poly f, int d, uint8_t* out) {
  memset(out, 0, 32 * d);
  int bit = 0;
  for (int i = 0; i < N; ++i)
    for (int b = 0; b < d; ++b, ++bit)
      out[bit >> 3] |= (uint8_t)(((f[i] >> b) & 1) << (bit & 7));
}
void byte_decode(const uint8_t* in, int d, poly f) {
  int bit = 0;
  for (int i = 0; i < N; ++i) {
    int v = 0;
    for (int b = 0; b < d; ++b, ++bit) v |= ((in[bit >> 3] >> (bit & 7)) & 1) << b;
    f[i] = (int16_t)v;
  }
}
inline int compress(int x, int d) { return (((x << d) + Q / 2) / Q) & ((1 << d) - 1); }
inline int decompress(int y, int d) { return (y * Q + (1 << (d - 1))) >> d; }

void sample_ntt(const uint8_t rho[32], uint8_t j, uint8_t i, poly a) {
  uint8_t seed[34];
  memcpy(seed, rho, 32); seed[32] = j; seed[33] = i;
  size_t want = 168 * 5;
  for (;;) {
    std::vector<uint8_t> buf(want);
    sx_shake128(seed, 34, buf.data(), want);
    int n = 0;
    for (size_t p = 0; p + 3 <= want && n < N; p += 3) {
      const int d1 = buf[p] | ((buf[p + 1] & 15) << 8), d2 = (buf[p + 1] >> 4) | (buf[p + 2] << 4);
      if (d1 < Q) a[n++] = (int16_t)d1;
      if (d2 < Q && n < N) a[n++] = (int16_t)d2;
    }
    if (n == N) return;
    want *= 2;   // the stream is a prefix-consistent XOF, so a longer squeeze repeats the same leading bytes
  }
}
void sample_cbd(const uint8_t seed[32], uint8_t nonce, int eta, poly f) {
  uint8_t in[33], buf[64 * 3];
  memcpy(in, seed, 32); in[32] = nonce;
  sx_shake256(in, 33, buf, 64 * eta);
  auto bit = [&](int i) { return (buf[i >> 3] >> (i & 7)) & 1; };
  for (int i = 0; i < N; ++i) {
    int x = 0, y = 0;
    for (int j = 0; j < eta; ++j) { x += bit(2 * i * eta + j); y += bit(2 * i * eta + eta + j); }
    f[i] = modq(x - y);
  }
}

void pke_keygen(const Params& P, const uint8_t d[32], uint8_t* ek, uint8_t* dk_pke) {
  uint8_t in[33], g[64];
  memcpy(in, d, 32); in[32] = (uint8_t)P.k;
  sx_sha3_512(in, 33, g);
  const uint8_t *rho = g, *sigma = g + 32;
  poly s[4], e[4], t;
  uint8_t nonce = 0;
  for (int i = 0; i < P.k; ++i) sample_cbd(sigma, nonce++, P.eta1, s[i]);
  for (int i = 0; i < P.k; ++i) sample_cbd(sigma, nonce++, P.eta1, e[i]);
  for (int i = 0; i < P.k; ++i) { ntt(s[i]); ntt(e[i]); }
  for (int i = 0; i < P.k; ++i) {
    memcpy(t, e[i], sizeof(poly));
    for (int j = 0; j < P.k; ++j) { poly a; sample_ntt(rho, (uint8_t)j, (uint8_t)i, a); mul_acc(t, a, s[j]); }
    byte_encode(t, 12, ek + 384 * i);
    byte_encode(s[i], 12, dk_pke + 384 * i);
  }
  memcpy(ek + 384 * P.k, rho, 32);
}

void pke_encrypt(const Params& P, const uint8_t* ek, const uint8_t m[32], const uint8_t r[32], uint8_t* c) {
  poly t[4], y[4], e1[4], e2, u, v, mu;
  const uint8_t* rho = ek + 384 * P.k;
  for (int i = 0; i < P.k; ++i) byte_decode(ek + 384 * i, 12, t[i]);
  uint8_t nonce = 0;
  for (int i = 0; i < P.k; ++i) sample_cbd(r, nonce++, P.eta1, y[i]);
  for (int i = 0; i < P.k; ++i) sample_cbd(r, nonce++, P.eta2, e1[i]);
  sample_cbd(r, nonce, P.eta2, e2);
  for (int i = 0; i < P.k; ++i) ntt(y[i]);
  for (int i = 0; i < P.k; ++i) {
    memset(u, 0, sizeof(poly));
    for (int j = 0; j < P.k; ++j) { poly a; sample_ntt(rho, (uint8_t)i, (uint8_t)j, a); mul_acc(u, a, y[j]); }   // A^T
    intt(u);
    for (int n = 0; n < N; ++n) u[n] = (int16_t)compress(modq(u[n] + e1[i][n]), P.du);
    byte_encode(u, P.du, c + 32 * P.du * i);
  }
  memset(v, 0, sizeof(poly));
  for (int j = 0; j < P.k; ++j) mul_acc(v, t[j], y[j]);
  intt(v);
  byte_decode(m, 1, mu);
  for (int n = 0; n < N; ++n) v[n] = (int16_t)compress(modq(v[n] + e2[n] + decompress(mu[n], 1)), P.dv);
  byte_encode(v, P.dv, c + 32 * P.du * P.k);
}

void pke_decrypt(const Params& P, const uint8_t* dk_pke, const uint8_t* c, uint8_t m[32]) {
  poly u, s, w, v;
  memset(w, 0, sizeof(poly));
  for (int i = 0; i < P.k; ++i) {
    byte_decode(c + 32 * P.du * i, P.du, u);
    for (int n = 0; n < N; ++n) u[n] = (int16_t)decompress(u[n], P.du);
    ntt(u);
    byte_decode(dk_pke + 384 * i, 12, s);
    for (int n = 0; n < N; ++n) s[n] = modq(s[n]);
    mul_acc(w, s, u);
  }
  intt(w);
  byte_decode(c + 32 * P.du * P.k, P.dv, v);
  for (int n = 0; n < N; ++n) w[n] = (int16_t)compress(modq(decompress(v[n], P.dv) - w[n]), 1);
  byte_encode(w, 1, m);
}

}  // namespace

SX_EXPORT int sx_mlkem_sizes(int k, int* ek, int* dk, int* ct) {
  Params P;
  if (!params_for(k, P)) return -1;
  *ek = 384 * k + 32; *dk = 768 * k + 96; *ct = 32 * (P.du * k + P.dv);
  return 0;
}

// Key pair from the two 32-byte seeds d and z (FIPS 203 ML-KEM.KeyGen_internal).
SX_EXPORT int sx_mlkem_keygen(int k, const uint8_t* d, const uint8_t* z, uint8_t* ek, uint8_t* dk) {
  Params P;
  if (!params_for(k, P)) return -1;
  init_tables();
  pke_keygen(P, d, ek, dk);
  const int eklen = 384 * k + 32;
  memcpy(dk + 384 * k, ek, eklen);
  sx_sha3_256(ek, eklen, dk + 384 * k + eklen);
  memcpy(dk + 384 * k + eklen + 32, z, 32);
  return 0;
}

// Ciphertext and 32-byte shared secret from the 32-byte message seed m. Returns -2 when the encapsulation key holds a
// coefficient outside [0, q) (the modulus check of FIPS 203 section 7.2).
SX_EXPORT int sx_mlkem_encaps(int k, const uint8_t* ek, const uint8_t* m, uint8_t* ct, uint8_t* ss) {
  Params P;
  if (!params_for(k, P)) return -1;
  init_tables();
  for (int i = 0; i < k; ++i) {
    poly t; byte_decode(ek + 384 * i, 12, t);
    for (int n = 0; n < N; ++n) if (t[n] >= Q) return -2;
  }
  uint8_t in[64], g[64];
  memcpy(in, m, 32);
  sx_sha3_256(ek, 384 * k + 32, in + 32);
  sx_sha3_512(in, 64, g);
  memcpy(ss, g, 32);
  pke_encrypt(P, ek, m, g + 32, ct);
  return 0;
}

// Shared secret from a ciphertext; a ciphertext that does not re-encrypt to itself yields the pseudo-random secret
// derived from z (implicit rejection), never an error.
SX_EXPORT int sx_mlkem_decaps(int k, const uint8_t* dk, const uint8_t* ct, uint8_t* ss) {
  Params P;
  if (!params_for(k, P)) return -1;
  init_tables();
  const int eklen = 384 * k + 32, ctlen = 32 * (P.du * k + P.dv);
  const uint8_t *ek = dk + 384 * k, *h = ek + eklen, *z = h + 32;
  uint8_t in[64], g[64];
  pke_decrypt(P, dk, ct, in);
  memcpy(in + 32, h, 32);
  sx_sha3_512(in, 64, g);
  std::vector<uint8_t> jin(32 + ctlen), c2(ctlen);
  memcpy(jin.data(), z, 32); memcpy(jin.data() + 32, ct, ctlen);
  uint8_t kbar[32];
  sx_shake256(jin.data(), jin.size(), kbar, 32);
  pke_encrypt(P, ek, in, g + 32, c2.data());
  uint8_t diff = 0;
  for (int i = 0; i < ctlen; ++i) diff |= (uint8_t)(ct[i] ^ c2[i]);
  const uint8_t mask = (uint8_t)(-(int)(diff != 0));
  for (int i = 0; i < 32; ++i) ss[i] = (uint8_t)((g[i] & ~mask) | (kbar[i] & mask));
  return 0;
}
