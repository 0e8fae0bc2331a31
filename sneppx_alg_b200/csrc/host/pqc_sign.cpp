// Post-quantum signatures: ML-DSA (FIPS 204, the standardised form of Dilithium) at parameter sets 44 / 65 / 87.
//
// Reference counterpart: security/crypto/post_quantum (Dilithium). Written from FIPS 204: the 256-point NTT over
// Z_8380417 with zeta = 1753, rejection sampling of the matrix and the secret vectors from SHAKE, Power2Round /
// Decompose / hints, the Fiat-Shamir-with-aborts signing loop and the packed encodings. The tests check key generation
// from a seed byte for byte, and signatures in both directions, against an independent implementation. Not hardened
// against timing side channels.
#include <cstdint>
#include <cstring>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" {
void sx_shake256(const void* msg, size_t len, void* out, size_t outlen);
void sx_shake128(const void* msg, size_t len, void* out, size_t outlen);
}

namespace {

constexpr int N = 256, D = 13;
constexpr int32_t Q = 8380417;
typedef int32_t poly[N];
typedef std::vector<uint8_t> bytes;

struct Params { int k, l, eta, tau, lambda, gamma1_bits, gamma2_div, beta, omega; };
bool params_for(int level, Params& p) {
  if (level == 44) p = {4, 4, 2, 39, 128, 17, 88, 78, 80};
  else if (level == 65) p = {6, 5, 4, 49, 192, 19, 32, 196, 55};
  else if (level == 87) p = {8, 7, 2, 60, 256, 19, 32, 120, 75};
  else return false;
  return true;
}
inline int32_t gamma1(const Params& p) { return 1 << p.gamma1_bits; }
inline int32_t gamma2(const Params& p) { return (Q - 1) / p.gamma2_div; }
inline int eta_bits(const Params& p) { return p.eta == 2 ? 3 : 4; }
inline int w1_bits(const Params& p) { return p.gamma2_div == 88 ? 6 : 4; }
inline int pk_len(const Params& p) { return 32 + 320 * p.k; }
inline int sk_len(const Params& p) { return 128 + 32 * ((p.l + p.k) * eta_bits(p) + D * p.k); }
inline int sig_len(const Params& p) { return p.lambda / 4 + p.l * 32 * (1 + p.gamma1_bits) + p.omega + p.k; }

int32_t zetas[256];
bool tables_ready = false;
void init_tables() {
  if (tables_ready) return;
  for (int m = 0; m < 256; ++m) {
    int br = 0;
    for (int b = 0; b < 8; ++b) br |= ((m >> b) & 1) << (7 - b);
    int64_t r = 1, x = 1753;
    for (int e = br; e; e >>= 1) { if (e & 1) r = r * x % Q; x = x * x % Q; }
    zetas[m] = (int32_t)r;
  }
  tables_ready = true;
}
inline int32_t modq(int64_t x) { int64_t r = x % Q; return (int32_t)(r < 0 ? r + Q : r); }
inline int32_t centered(int32_t x) { return x > (Q - 1) / 2 ? x - Q : x; }   // x in [0, q)

void ntt(poly w) {
  int m = 0;
  for (int len = 128; len >= 1; len >>= 1)
    for (int start = 0; start < N; start += 2 * len) {
      const int64_t z = zetas[++m];
      for (int j = start; j < start + len; ++j) {
        const int32_t t = modq(z * w[j + len]);
        w[j + len] = modq((int64_t)w[j] - t);
        w[j] = modq((int64_t)w[j] + t);
      }
    }
}
void intt(poly w) {
  int m = 256;
  for (int len = 1; len < N; len <<= 1)
    for (int start = 0; start < N; start += 2 * len) {
      const int64_t z = -(int64_t)zetas[--m];
      for (int j = start; j < start + len; ++j) {
        const int32_t t = w[j];
        w[j] = modq((int64_t)t + w[j + len]);
        w[j + len] = modq(z * modq((int64_t)t - w[j + len]));
      }
    }
  for (int j = 0; j < N; ++j) w[j] = modq((int64_t)w[j] * 8347681);   // 256^-1 mod q
}
inline void pointwise_acc(poly acc, const poly a, const poly b) {
  for (int i = 0; i < N; ++i) acc[i] = modq(acc[i] + (int64_t)a[i] * b[i]);
}
inline void pointwise(poly out, const poly a, const poly b) {
  for (int i = 0; i < N; ++i) out[i] = modq((int64_t)a[i] * b[i]);
}

// ----------------------------------------------------------------------------------------------- bit packing
struct BitWriter {
  uint8_t* p; int bit = 0;
  explicit BitWriter(uint8_t* out) : p(out) {}
  void put(uint32_t v, int nbits) { for (int b = 0; b < nbits; ++b, ++bit) { if (!(bit & 7)) p[bit >> 3] = 0; p[bit >> 3] |= (uint8_t)(((v >> b) & 1) << (bit & 7)); } }
};
struct BitReader {
  const uint8_t* p; int bit = 0;
  explicit BitReader(const uint8_t* in) : p(in) {}
  uint32_t get(int nbits) { uint32_t v = 0; for (int b = 0; b < nbits; ++b, ++bit) v |= (uint32_t)((p[bit >> 3] >> (bit & 7)) & 1) << b; return v; }
};
// coefficients in [-a, b] stored as b - w in `nbits` bits; polynomials hold values mod q
void pack_signed(const poly w, int32_t b, int nbits, uint8_t* out) {
  BitWriter bw(out);
  for (int i = 0; i < N; ++i) bw.put((uint32_t)(b - centered(w[i])), nbits);
}
void unpack_signed(const uint8_t* in, int32_t b, int nbits, poly w) {
  BitReader br(in);
  for (int i = 0; i < N; ++i) w[i] = modq((int64_t)b - (int64_t)br.get(nbits));
}
void pack_unsigned(const poly w, int nbits, uint8_t* out) { BitWriter bw(out); for (int i = 0; i < N; ++i) bw.put((uint32_t)w[i], nbits); }
void unpack_unsigned(const uint8_t* in, int nbits, poly w) { BitReader br(in); for (int i = 0; i < N; ++i) w[i] = (int32_t)br.get(nbits); }

// ----------------------------------------------------------------------------------------------- sampling
void rej_ntt_poly(const uint8_t rho[32], uint8_t s, uint8_t r, poly a) {
  uint8_t seed[34];
  memcpy(seed, rho, 32); seed[32] = s; seed[33] = r;
  for (size_t want = 168 * 6;; want *= 2) {
    bytes buf(want);
    sx_shake128(seed, 34, buf.data(), want);
    int n = 0;
    for (size_t p = 0; p + 3 <= want && n < N; p += 3) {
      const int32_t z = buf[p] | (buf[p + 1] << 8) | ((buf[p + 2] & 127) << 16);
      if (z < Q) a[n++] = z;
    }
    if (n == N) return;
  }
}
void rej_bounded_poly(const uint8_t rhop[64], uint16_t r, int eta, poly a) {
  uint8_t seed[66];
  memcpy(seed, rhop, 64); seed[64] = (uint8_t)r; seed[65] = (uint8_t)(r >> 8);
  for (size_t want = 136 * 4;; want *= 2) {
    bytes buf(want);
    sx_shake256(seed, 66, buf.data(), want);
    int n = 0;
    for (size_t p = 0; p < want && n < N; ++p)
      for (int half = 0; half < 2 && n < N; ++half) {
        const int b = half ? buf[p] >> 4 : buf[p] & 15;
        if (eta == 2 && b < 15) a[n++] = modq(2 - (b % 5));
        else if (eta == 4 && b < 9) a[n++] = modq(4 - b);
      }
    if (n == N) return;
  }
}
void sample_in_ball(const uint8_t* ctilde, int len, int tau, poly c) {
  memset(c, 0, sizeof(poly));
  for (size_t want = 8 + 512;; want *= 2) {
    bytes buf(want);
    sx_shake256(ctilde, len, buf.data(), want);
    uint64_t signs; memcpy(&signs, buf.data(), 8);
    size_t pos = 8;
    bool ok = true;
    memset(c, 0, sizeof(poly));
    for (int i = N - tau; i < N && ok; ++i) {
      int j;
      do { if (pos >= want) { ok = false; break; } j = buf[pos++]; } while (j > i);
      if (!ok) break;
      c[i] = c[j];
      c[j] = ((signs >> (i + tau - N)) & 1) ? Q - 1 : 1;
    }
    if (ok) return;
  }
}
void expand_mask(const Params& P, const uint8_t rho2[64], int kappa, poly* y) {
  const int c = 1 + P.gamma1_bits;
  uint8_t seed[66];
  memcpy(seed, rho2, 64);
  bytes v(32 * c);
  for (int r = 0; r < P.l; ++r) {
    const int n = kappa + r;
    seed[64] = (uint8_t)n; seed[65] = (uint8_t)(n >> 8);
    sx_shake256(seed, 66, v.data(), v.size());
    unpack_signed(v.data(), gamma1(P), c, y[r]);
  }
}

// ----------------------------------------------------------------------------------------------- rounding
inline void power2round(int32_t r, int32_t& r1, int32_t& r0) {
  r0 = r & ((1 << D) - 1);
  if (r0 > (1 << (D - 1))) r0 -= 1 << D;
  r1 = (r - r0) >> D;
}
inline void decompose(const Params& P, int32_t r, int32_t& r1, int32_t& r0) {
  const int32_t g2 = 2 * gamma2(P);
  r0 = r % g2;
  if (r0 > g2 / 2) r0 -= g2;
  if (r - r0 == Q - 1) { r1 = 0; r0 -= 1; } else r1 = (r - r0) / g2;
}
inline int32_t high_bits(const Params& P, int32_t r) { int32_t r1, r0; decompose(P, r, r1, r0); return r1; }
inline int32_t use_hint(const Params& P, int h, int32_t r) {
  const int32_t m = (Q - 1) / (2 * gamma2(P));
  int32_t r1, r0; decompose(P, r, r1, r0);
  if (!h) return r1;
  return r0 > 0 ? (r1 + 1) % m : (r1 - 1 + m) % m;
}
inline int32_t inf_norm(const poly w) { int32_t m = 0; for (int i = 0; i < N; ++i) { int32_t a = centered(w[i]); if (a < 0) a = -a; if (a > m) m = a; } return m; }

bytes shake256_cat(const uint8_t* a, size_t alen, const uint8_t* b, size_t blen, const uint8_t* c, size_t clen, size_t outlen) {
  bytes in(alen + blen + clen), out(outlen);
  if (alen) memcpy(in.data(), a, alen);
  if (blen) memcpy(in.data() + alen, b, blen);
  if (clen) memcpy(in.data() + alen + blen, c, clen);
  sx_shake256(in.data(), in.size(), out.data(), outlen);
  return out;
}
// mu = H(H(pk) || 0 || |ctx| || ctx || M)
bytes message_digest(const uint8_t tr[64], const uint8_t* msg, size_t mlen, const uint8_t* ctx, size_t clen) {
  bytes in(64 + 2 + clen + mlen), out(64);
  memcpy(in.data(), tr, 64);
  in[64] = 0; in[65] = (uint8_t)clen;
  if (clen) memcpy(in.data() + 66, ctx, clen);
  if (mlen) memcpy(in.data() + 66 + clen, msg, mlen);
  sx_shake256(in.data(), in.size(), out.data(), 64);
  return out;
}

}  // namespace

SX_EXPORT int sx_mldsa_sizes(int level, int* pk, int* sk, int* sig) {
  Params P;
  if (!params_for(level, P)) return -1;
  *pk = pk_len(P); *sk = sk_len(P); *sig = sig_len(P);
  return 0;
}

// Key pair from a 32-byte seed (FIPS 204 ML-DSA.KeyGen_internal).
SX_EXPORT int sx_mldsa_keygen(int level, const uint8_t* xi, uint8_t* pk, uint8_t* sk) {
  Params P;
  if (!params_for(level, P)) return -1;
  init_tables();
  uint8_t in[34], h[128];
  memcpy(in, xi, 32); in[32] = (uint8_t)P.k; in[33] = (uint8_t)P.l;
  sx_shake256(in, 34, h, 128);
  const uint8_t *rho = h, *rhop = h + 32, *K = h + 96;
  std::vector<int32_t> store((size_t)(2 * P.l + 2 * P.k) * N);
  poly* s1 = (poly*)store.data(); poly* s1h = s1 + P.l; poly* s2 = s1h + P.l; poly* t = s2 + P.k;
  for (int r = 0; r < P.l; ++r) { rej_bounded_poly(rhop, (uint16_t)r, P.eta, s1[r]); memcpy(s1h[r], s1[r], sizeof(poly)); ntt(s1h[r]); }
  for (int r = 0; r < P.k; ++r) rej_bounded_poly(rhop, (uint16_t)(r + P.l), P.eta, s2[r]);
  memcpy(pk, rho, 32);
  uint8_t* skp = sk;
  memcpy(skp, rho, 32); memcpy(skp + 32, K, 32); skp += 128;   // tr is filled in once pk is complete
  const int eb = eta_bits(P);
  for (int r = 0; r < P.l; ++r, skp += 32 * eb) pack_signed(s1[r], P.eta, eb, skp);
  for (int r = 0; r < P.k; ++r, skp += 32 * eb) pack_signed(s2[r], P.eta, eb, skp);
  for (int r = 0; r < P.k; ++r) {
    memset(t[r], 0, sizeof(poly));
    for (int s = 0; s < P.l; ++s) { poly a; rej_ntt_poly(rho, (uint8_t)s, (uint8_t)r, a); pointwise_acc(t[r], a, s1h[s]); }
    intt(t[r]);
    poly t1, t0;
    for (int i = 0; i < N; ++i) { int32_t hi, lo; power2round(modq((int64_t)t[r][i] + s2[r][i]), hi, lo); t1[i] = hi; t0[i] = modq(lo); }
    pack_unsigned(t1, 10, pk + 32 + 320 * r);
    pack_signed(t0, 1 << (D - 1), D, skp); skp += 32 * D;
  }
  sx_shake256(pk, pk_len(P), sk + 64, 64);
  return 0;
}

// Signature over `msg` with context string `ctx` (at most 255 bytes). `rnd` is 32 bytes: fresh randomness for the
// hedged variant, zeros for the deterministic one. Returns 0, or -1 on bad arguments.
SX_EXPORT int sx_mldsa_sign(int level, const uint8_t* sk, const uint8_t* msg, size_t mlen, const uint8_t* ctx, size_t clen,
                            const uint8_t* rnd, uint8_t* sig) {
  Params P;
  if (!params_for(level, P) || clen > 255) return -1;
  init_tables();
  const uint8_t *rho = sk, *K = sk + 32, *tr = sk + 64;
  const int eb = eta_bits(P), clen_t = P.lambda / 4, zbits = 1 + P.gamma1_bits;
  std::vector<int32_t> store((size_t)(P.l * (P.k + 4) + 5 * P.k) * N);
  poly* A = (poly*)store.data();          // k x l, NTT domain
  poly* s1 = A + P.k * P.l; poly* s2 = s1 + P.l; poly* t0 = s2 + P.k;
  poly* y = t0 + P.k; poly* yh = y + P.l; poly* z = yh + P.l; poly* w = z + P.l; poly* wcs2 = w + P.k;
  const uint8_t* p = sk + 128;
  for (int r = 0; r < P.l; ++r, p += 32 * eb) { unpack_signed(p, P.eta, eb, s1[r]); ntt(s1[r]); }
  for (int r = 0; r < P.k; ++r, p += 32 * eb) { unpack_signed(p, P.eta, eb, s2[r]); ntt(s2[r]); }
  for (int r = 0; r < P.k; ++r, p += 32 * D) { unpack_signed(p, 1 << (D - 1), D, t0[r]); ntt(t0[r]); }
  for (int r = 0; r < P.k; ++r) for (int s = 0; s < P.l; ++s) rej_ntt_poly(rho, (uint8_t)s, (uint8_t)r, A[r * P.l + s]);
  const bytes mu = message_digest(tr, msg, mlen, ctx, clen);
  const bytes rho2 = shake256_cat(K, 32, rnd, 32, mu.data(), 64, 64);
  const int32_t g1 = gamma1(P), g2 = gamma2(P);
  bytes w1enc(32 * w1_bits(P) * P.k), hint(P.omega + P.k);
  for (int kappa = 0; kappa < 1 << 16; kappa += P.l) {
    expand_mask(P, rho2.data(), kappa, y);
    for (int s = 0; s < P.l; ++s) { memcpy(yh[s], y[s], sizeof(poly)); ntt(yh[s]); }
    for (int r = 0; r < P.k; ++r) {
      memset(w[r], 0, sizeof(poly));
      for (int s = 0; s < P.l; ++s) pointwise_acc(w[r], A[r * P.l + s], yh[s]);
      intt(w[r]);
      poly w1;
      for (int i = 0; i < N; ++i) w1[i] = high_bits(P, w[r][i]);
      pack_unsigned(w1, w1_bits(P), w1enc.data() + 32 * w1_bits(P) * r);
    }
    const bytes ctilde = shake256_cat(mu.data(), 64, w1enc.data(), w1enc.size(), nullptr, 0, clen_t);
    poly c, t;
    sample_in_ball(ctilde.data(), clen_t, P.tau, c);
    ntt(c);
    bool reject = false;
    for (int s = 0; s < P.l && !reject; ++s) {
      pointwise(t, c, s1[s]); intt(t);
      for (int i = 0; i < N; ++i) z[s][i] = modq((int64_t)y[s][i] + t[i]);
      reject = inf_norm(z[s]) >= g1 - P.beta;
    }
    for (int r = 0; r < P.k && !reject; ++r) {
      pointwise(t, c, s2[r]); intt(t);
      for (int i = 0; i < N; ++i) {
        wcs2[r][i] = modq((int64_t)w[r][i] - t[i]);
        int32_t r1, r0; decompose(P, wcs2[r][i], r1, r0);
        if (r0 >= g2 - P.beta || -r0 >= g2 - P.beta) reject = true;
      }
    }
    if (reject) continue;
    int ones = 0;
    memset(hint.data(), 0, hint.size());
    for (int r = 0; r < P.k && !reject; ++r) {
      pointwise(t, c, t0[r]); intt(t);
      if (inf_norm(t) >= g2) { reject = true; break; }
      for (int i = 0; i < N; ++i) {
        // hint bit: does adding c*t0 back change the high bits of w - c*s2 ?
        const int32_t with = modq((int64_t)wcs2[r][i] + t[i]);
        if (high_bits(P, wcs2[r][i]) != high_bits(P, with)) {
          if (ones >= P.omega) { reject = true; break; }
          hint[ones++] = (uint8_t)i;
        }
      }
      hint[P.omega + r] = (uint8_t)ones;
    }
    if (reject) continue;
    memcpy(sig, ctilde.data(), clen_t);
    uint8_t* q = sig + clen_t;
    for (int s = 0; s < P.l; ++s, q += 32 * zbits) pack_signed(z[s], g1, zbits, q);
    memcpy(q, hint.data(), hint.size());
    return 0;
  }
  return -1;
}

// 1 when `sig` is a valid signature of `msg` under `pk` and context `ctx`, else 0.
SX_EXPORT int sx_mldsa_verify(int level, const uint8_t* pk, const uint8_t* msg, size_t mlen, const uint8_t* ctx, size_t clen,
                              const uint8_t* sig) {
  Params P;
  if (!params_for(level, P) || clen > 255) return 0;
  init_tables();
  const int clen_t = P.lambda / 4, zbits = 1 + P.gamma1_bits;
  const uint8_t* rho = pk;
  std::vector<int32_t> store((size_t)(P.l + 1) * N);
  poly* z = (poly*)store.data();
  const uint8_t* q = sig + clen_t;
  for (int s = 0; s < P.l; ++s, q += 32 * zbits) {
    unpack_signed(q, gamma1(P), zbits, z[s]);
    if (inf_norm(z[s]) >= gamma1(P) - P.beta) return 0;
    ntt(z[s]);
  }
  // hints: omega positions followed by k running totals; positions strictly increase within a row, unused tail is 0
  std::vector<uint8_t> h((size_t)P.k * N, 0);
  int index = 0;
  for (int r = 0; r < P.k; ++r) {
    const int end = q[P.omega + r];
    if (end < index || end > P.omega) return 0;
    const int first = index;
    for (; index < end; ++index) {
      if (index > first && q[index - 1] >= q[index]) return 0;
      h[(size_t)r * N + q[index]] = 1;
    }
  }
  for (int i = index; i < P.omega; ++i) if (q[i]) return 0;
  uint8_t tr[64];
  sx_shake256(pk, pk_len(P), tr, 64);
  const bytes mu = message_digest(tr, msg, mlen, ctx, clen);
  poly c, t1, acc, a;
  sample_in_ball(sig, clen_t, P.tau, c);
  ntt(c);
  bytes w1enc(32 * w1_bits(P) * P.k);
  for (int r = 0; r < P.k; ++r) {
    memset(acc, 0, sizeof(poly));
    for (int s = 0; s < P.l; ++s) { rej_ntt_poly(rho, (uint8_t)s, (uint8_t)r, a); pointwise_acc(acc, a, z[s]); }
    unpack_unsigned(pk + 32 + 320 * r, 10, t1);
    for (int i = 0; i < N; ++i) t1[i] = (int32_t)(((int64_t)t1[i] << D) % Q);
    ntt(t1);
    for (int i = 0; i < N; ++i) acc[i] = modq((int64_t)acc[i] - (int64_t)c[i] * t1[i]);
    intt(acc);
    poly w1;
    for (int i = 0; i < N; ++i) w1[i] = use_hint(P, h[(size_t)r * N + i], acc[i]);
    pack_unsigned(w1, w1_bits(P), w1enc.data() + 32 * w1_bits(P) * r);
  }
  const bytes c2 = shake256_cat(mu.data(), 64, w1enc.data(), w1enc.size(), nullptr, 0, clen_t);
  uint8_t diff = 0;
  for (int i = 0; i < clen_t; ++i) diff |= (uint8_t)(c2[i] ^ sig[i]);
  return diff == 0;
}
