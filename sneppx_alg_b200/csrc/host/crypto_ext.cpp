// Further S0 primitives: SHA-512, SHA-3 / SHAKE (Keccak-f[1600]), BLAKE2b, AES-256-GCM and Ed25519 signatures.
//
// Reference counterparts: security/crypto/c (sha2, sha3, blake, aes_gcm, ed25519 and the bignum helpers). Written from
// the public specifications (FIPS 180-4, FIPS 202, RFC 7693, FIPS 197 + SP 800-38D, RFC 8032) and checked against
// their published vectors and against independent implementations in the tests. Host-side utilities for signed
// updates, audit chains and the key vault; the scalar arithmetic is not hardened against timing side channels.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

inline uint64_t rotr64(uint64_t x, int n) { return (x >> n) | (x << (64 - n)); }
inline uint64_t rotl64(uint64_t x, int n) { return n ? (x << n) | (x >> (64 - n)) : x; }

// ------------------------------------------------------------------------------------------------ SHA-512
const uint64_t K512[80] = {
    0x428a2f98d728ae22ULL, 0x7137449123ef65cdULL, 0xb5c0fbcfec4d3b2fULL, 0xe9b5dba58189dbbcULL, 0x3956c25bf348b538ULL,
    0x59f111f1b605d019ULL, 0x923f82a4af194f9bULL, 0xab1c5ed5da6d8118ULL, 0xd807aa98a3030242ULL, 0x12835b0145706fbeULL,
    0x243185be4ee4b28cULL, 0x550c7dc3d5ffb4e2ULL, 0x72be5d74f27b896fULL, 0x80deb1fe3b1696b1ULL, 0x9bdc06a725c71235ULL,
    0xc19bf174cf692694ULL, 0xe49b69c19ef14ad2ULL, 0xefbe4786384f25e3ULL, 0x0fc19dc68b8cd5b5ULL, 0x240ca1cc77ac9c65ULL,
    0x2de92c6f592b0275ULL, 0x4a7484aa6ea6e483ULL, 0x5cb0a9dcbd41fbd4ULL, 0x76f988da831153b5ULL, 0x983e5152ee66dfabULL,
    0xa831c66d2db43210ULL, 0xb00327c898fb213fULL, 0xbf597fc7beef0ee4ULL, 0xc6e00bf33da88fc2ULL, 0xd5a79147930aa725ULL,
    0x06ca6351e003826fULL, 0x142929670a0e6e70ULL, 0x27b70a8546d22ffcULL, 0x2e1b21385c26c926ULL, 0x4d2c6dfc5ac42aedULL,
    0x53380d139d95b3dfULL, 0x650a73548baf63deULL, 0x766a0abb3c77b2a8ULL, 0x81c2c92e47edaee6ULL, 0x92722c851482353bULL,
    0xa2bfe8a14cf10364ULL, 0xa81a664bbc423001ULL, 0xc24b8b70d0f89791ULL, 0xc76c51a30654be30ULL, 0xd192e819d6ef5218ULL,
    0xd69906245565a910ULL, 0xf40e35855771202aULL, 0x106aa07032bbd1b8ULL, 0x19a4c116b8d2d0c8ULL, 0x1e376c085141ab53ULL,
    0x2748774cdf8eeb99ULL, 0x34b0bcb5e19b48a8ULL, 0x391c0cb3c5c95a63ULL, 0x4ed8aa4ae3418acbULL, 0x5b9cca4f7763e373ULL,
    0x682e6ff3d6b2b8a3ULL, 0x748f82ee5defb2fcULL, 0x78a5636f43172f60ULL, 0x84c87814a1f0ab72ULL, 0x8cc702081a6439ecULL,
    0x90befffa23631e28ULL, 0xa4506cebde82bde9ULL, 0xbef9a3f7b2c67915ULL, 0xc67178f2e372532bULL, 0xca273eceea26619cULL,
    0xd186b8c721c0c207ULL, 0xeada7dd6cde0eb1eULL, 0xf57d4f7fee6ed178ULL, 0x06f067aa72176fbaULL, 0x0a637dc5a2c898a6ULL,
    0x113f9804bef90daeULL, 0x1b710b35131c471bULL, 0x28db77f523047d84ULL, 0x32caab7b40c72493ULL, 0x3c9ebe0a15c9bebcULL,
    0x431d67c49c100d4cULL, 0x4cc5d4becb3e42b6ULL, 0x597f299cfc657e2aULL, 0x5fcb6fab3ad6faecULL, 0x6c44198c4a475817ULL};

void sha512(const uint8_t* msg, size_t len, uint8_t out[64]) {
  uint64_t h[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                   0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};
  std::vector<uint8_t> m(msg, msg + len);
  m.push_back(0x80);
  while (m.size() % 128 != 112) m.push_back(0);
  for (int i = 0; i < 8; ++i) m.push_back(0);  // high 64 bits of the length
  uint64_t bits = (uint64_t)len * 8;
  for (int i = 7; i >= 0; --i) m.push_back((uint8_t)(bits >> (8 * i)));
  for (size_t off = 0; off < m.size(); off += 128) {
    uint64_t w[80];
    for (int i = 0; i < 16; ++i) { w[i] = 0; for (int j = 0; j < 8; ++j) w[i] = w[i] << 8 | m[off + 8 * i + j]; }
    for (int i = 16; i < 80; ++i) {
      uint64_t s0 = rotr64(w[i - 15], 1) ^ rotr64(w[i - 15], 8) ^ (w[i - 15] >> 7);
      uint64_t s1 = rotr64(w[i - 2], 19) ^ rotr64(w[i - 2], 61) ^ (w[i - 2] >> 6);
      w[i] = w[i - 16] + s0 + w[i - 7] + s1;
    }
    uint64_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
    for (int i = 0; i < 80; ++i) {
      uint64_t S1 = rotr64(e, 14) ^ rotr64(e, 18) ^ rotr64(e, 41), ch = (e & f) ^ (~e & g);
      uint64_t t1 = hh + S1 + ch + K512[i] + w[i];
      uint64_t S0 = rotr64(a, 28) ^ rotr64(a, 34) ^ rotr64(a, 39), mj = (a & b) ^ (a & c) ^ (b & c);
      uint64_t t2 = S0 + mj;
      hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
    }
    h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
  }
  for (int i = 0; i < 8; ++i) for (int j = 0; j < 8; ++j) out[8 * i + j] = (uint8_t)(h[i] >> (56 - 8 * j));
}

// ------------------------------------------------------------------------------------------------ Keccak
void keccak_f(uint64_t s[25]) {
  static const int rot[25] = {0, 1, 62, 28, 27, 36, 44, 6, 55, 20, 3, 10, 43, 25, 39, 41, 45, 15, 21, 8, 18, 2, 61, 56, 14};
  uint64_t rc = 1;  // round constants from the degree-8 LFSR of FIPS 202, section 3.2.5
  auto lfsr_bit = [](uint8_t& r) { bool bit = r & 1; r = (r & 0x80) ? (uint8_t)((r << 1) ^ 0x71) : (uint8_t)(r << 1); return bit; };
  uint8_t r = 1;
  for (int round = 0; round < 24; ++round) {
    uint64_t c[5], d[5], b[25];
    for (int x = 0; x < 5; ++x) c[x] = s[x] ^ s[x + 5] ^ s[x + 10] ^ s[x + 15] ^ s[x + 20];
    for (int x = 0; x < 5; ++x) d[x] = c[(x + 4) % 5] ^ rotl64(c[(x + 1) % 5], 1);
    for (int i = 0; i < 25; ++i) s[i] ^= d[i % 5];
    for (int x = 0; x < 5; ++x) for (int y = 0; y < 5; ++y) b[y + 5 * ((2 * x + 3 * y) % 5)] = rotl64(s[x + 5 * y], rot[x + 5 * y]);
    for (int y = 0; y < 5; ++y) for (int x = 0; x < 5; ++x) s[x + 5 * y] = b[x + 5 * y] ^ (~b[(x + 1) % 5 + 5 * y] & b[(x + 2) % 5 + 5 * y]);
    rc = 0;
    for (int j = 0; j < 7; ++j) if (lfsr_bit(r)) rc |= 1ULL << ((1 << j) - 1);
    s[0] ^= rc;
  }
}

void keccak(const uint8_t* msg, size_t len, size_t rate, uint8_t suffix, uint8_t* out, size_t outlen) {
  uint64_t s[25] = {0};
  auto absorb_block = [&](const uint8_t* p) { for (size_t i = 0; i < rate / 8; ++i) { uint64_t v; memcpy(&v, p + 8 * i, 8); s[i] ^= v; } keccak_f(s); };
  while (len >= rate) { absorb_block(msg); msg += rate; len -= rate; }
  std::vector<uint8_t> last(rate, 0);
  memcpy(last.data(), msg, len);
  last[len] ^= suffix;
  last[rate - 1] ^= 0x80;
  absorb_block(last.data());
  while (outlen) {
    size_t n = outlen < rate ? outlen : rate;
    memcpy(out, s, n);
    out += n; outlen -= n;
    if (outlen) keccak_f(s);
  }
}

// ------------------------------------------------------------------------------------------------ BLAKE2b
const uint8_t B2_SIGMA[12][16] = {
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3},
    {11, 8, 12, 0, 5, 2, 15, 13, 10, 14, 3, 6, 7, 1, 9, 4}, {7, 9, 3, 1, 13, 12, 11, 14, 2, 6, 5, 10, 4, 0, 15, 8},
    {9, 0, 5, 7, 2, 4, 10, 15, 14, 1, 11, 12, 6, 8, 3, 13}, {2, 12, 6, 10, 0, 11, 8, 3, 4, 13, 7, 5, 15, 14, 1, 9},
    {12, 5, 1, 15, 14, 13, 4, 10, 0, 7, 6, 3, 9, 2, 8, 11}, {13, 11, 7, 14, 12, 1, 3, 9, 5, 0, 15, 4, 8, 6, 2, 10},
    {6, 15, 14, 9, 11, 3, 0, 8, 12, 2, 13, 7, 1, 4, 10, 5}, {10, 2, 8, 4, 7, 6, 1, 5, 15, 11, 9, 14, 3, 12, 13, 0},
    {0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15}, {14, 10, 4, 8, 9, 15, 13, 6, 1, 12, 0, 2, 11, 7, 5, 3}};
const uint64_t B2_IV[8] = {0x6a09e667f3bcc908ULL, 0xbb67ae8584caa73bULL, 0x3c6ef372fe94f82bULL, 0xa54ff53a5f1d36f1ULL,
                           0x510e527fade682d1ULL, 0x9b05688c2b3e6c1fULL, 0x1f83d9abfb41bd6bULL, 0x5be0cd19137e2179ULL};

void blake2b_compress(uint64_t h[8], const uint8_t block[128], uint64_t t, bool last) {
  uint64_t m[16], v[16];
  for (int i = 0; i < 16; ++i) memcpy(&m[i], block + 8 * i, 8);
  for (int i = 0; i < 8; ++i) { v[i] = h[i]; v[i + 8] = B2_IV[i]; }
  v[12] ^= t;
  if (last) v[14] = ~v[14];
  auto G = [&](int a, int b, int c, int d, uint64_t x, uint64_t y) {
    v[a] = v[a] + v[b] + x; v[d] = rotr64(v[d] ^ v[a], 32); v[c] = v[c] + v[d]; v[b] = rotr64(v[b] ^ v[c], 24);
    v[a] = v[a] + v[b] + y; v[d] = rotr64(v[d] ^ v[a], 16); v[c] = v[c] + v[d]; v[b] = rotr64(v[b] ^ v[c], 63);
  };
  for (int r = 0; r < 12; ++r) {
    const uint8_t* s = B2_SIGMA[r];
    G(0, 4, 8, 12, m[s[0]], m[s[1]]); G(1, 5, 9, 13, m[s[2]], m[s[3]]); G(2, 6, 10, 14, m[s[4]], m[s[5]]); G(3, 7, 11, 15, m[s[6]], m[s[7]]);
    G(0, 5, 10, 15, m[s[8]], m[s[9]]); G(1, 6, 11, 12, m[s[10]], m[s[11]]); G(2, 7, 8, 13, m[s[12]], m[s[13]]); G(3, 4, 9, 14, m[s[14]], m[s[15]]);
  }
  for (int i = 0; i < 8; ++i) h[i] ^= v[i] ^ v[i + 8];
}

int blake2b(const uint8_t* msg, size_t len, const uint8_t* key, size_t keylen, uint8_t* out, size_t outlen) {
  if (outlen == 0 || outlen > 64 || keylen > 64) return -1;
  uint64_t h[8];
  memcpy(h, B2_IV, sizeof h);
  h[0] ^= 0x01010000ULL ^ ((uint64_t)keylen << 8) ^ (uint64_t)outlen;
  std::vector<uint8_t> data;
  if (keylen) { data.assign(128, 0); memcpy(data.data(), key, keylen); }
  data.insert(data.end(), msg, msg + len);
  if (data.empty()) data.assign(128, 0), len = 0;
  size_t total = keylen ? 128 + len : len, off = 0;
  while (total - off > 128) { blake2b_compress(h, data.data() + off, off + 128, false); off += 128; }
  uint8_t last[128] = {0};
  memcpy(last, data.data() + off, total - off);
  blake2b_compress(h, last, total, true);
  memcpy(out, h, outlen);
  return 0;
}

}  // namespace

SX_EXPORT void sx_sha512(const void* msg, size_t len, void* out64) { sha512((const uint8_t*)msg, len, (uint8_t*)out64); }
SX_EXPORT void sx_sha3_256(const void* msg, size_t len, void* out32) { keccak((const uint8_t*)msg, len, 136, 0x06, (uint8_t*)out32, 32); }
SX_EXPORT void sx_sha3_512(const void* msg, size_t len, void* out64) { keccak((const uint8_t*)msg, len, 72, 0x06, (uint8_t*)out64, 64); }
SX_EXPORT void sx_shake128(const void* msg, size_t len, void* out, size_t outlen) { keccak((const uint8_t*)msg, len, 168, 0x1F, (uint8_t*)out, outlen); }
SX_EXPORT void sx_shake256(const void* msg, size_t len, void* out, size_t outlen) { keccak((const uint8_t*)msg, len, 136, 0x1F, (uint8_t*)out, outlen); }
SX_EXPORT int sx_blake2b(const void* msg, size_t len, const void* key, size_t keylen, void* out, size_t outlen) {
  return blake2b((const uint8_t*)msg, len, (const uint8_t*)key, keylen, (uint8_t*)out, outlen);
}

// ------------------------------------------------------------------------------------------------ AES-256-GCM
namespace {

struct AesTables {
  uint8_t sbox[256];
  AesTables() {
    // S-box = affine map of the multiplicative inverse in GF(2^8) mod x^8 + x^4 + x^3 + x + 1 (FIPS 197, 5.1.1)
    auto mul = [](uint8_t a, uint8_t b) { uint8_t p = 0; for (int i = 0; i < 8; ++i) { if (b & 1) p ^= a; bool hi = a & 0x80; a <<= 1; if (hi) a ^= 0x1B; b >>= 1; } return p; };
    for (int x = 0; x < 256; ++x) {
      uint8_t inv = 0;
      if (x) for (int y = 1; y < 256; ++y) if (mul((uint8_t)x, (uint8_t)y) == 1) { inv = (uint8_t)y; break; }
      uint8_t s = inv;
      for (int i = 1; i <= 4; ++i) s ^= (uint8_t)((inv << i) | (inv >> (8 - i)));
      sbox[x] = s ^ 0x63;
    }
  }
};
const AesTables& aes_tables() { static AesTables t; return t; }

struct Aes256 {
  uint8_t rk[15][16];
  explicit Aes256(const uint8_t key[32]) {
    const uint8_t* S = aes_tables().sbox;
    uint8_t w[60][4];
    memcpy(w, key, 32);
    uint8_t rcon = 1;
    for (int i = 8; i < 60; ++i) {
      uint8_t t[4] = {w[i - 1][0], w[i - 1][1], w[i - 1][2], w[i - 1][3]};
      if (i % 8 == 0) {
        uint8_t u = t[0]; t[0] = S[t[1]] ^ rcon; t[1] = S[t[2]]; t[2] = S[t[3]]; t[3] = S[u];
        rcon = (uint8_t)((rcon << 1) ^ ((rcon & 0x80) ? 0x1B : 0));
      } else if (i % 8 == 4) for (int j = 0; j < 4; ++j) t[j] = S[t[j]];
      for (int j = 0; j < 4; ++j) w[i][j] = w[i - 8][j] ^ t[j];
    }
    memcpy(rk, w, sizeof rk);
  }
  void encrypt(const uint8_t in[16], uint8_t out[16]) const {
    const uint8_t* S = aes_tables().sbox;
    uint8_t s[16];
    for (int i = 0; i < 16; ++i) s[i] = in[i] ^ rk[0][i];
    auto xt = [](uint8_t a) { return (uint8_t)((a << 1) ^ ((a & 0x80) ? 0x1B : 0)); };
    for (int r = 1; r <= 14; ++r) {
      uint8_t t[16];
      for (int c = 0; c < 4; ++c) for (int row = 0; row < 4; ++row) t[4 * c + row] = S[s[4 * ((c + row) % 4) + row]];  // SubBytes + ShiftRows
      if (r < 14) for (int c = 0; c < 4; ++c) {
        uint8_t* col = t + 4 * c;
        uint8_t a0 = col[0], a1 = col[1], a2 = col[2], a3 = col[3], all = a0 ^ a1 ^ a2 ^ a3;
        col[0] = a0 ^ all ^ xt(a0 ^ a1); col[1] = a1 ^ all ^ xt(a1 ^ a2); col[2] = a2 ^ all ^ xt(a2 ^ a3); col[3] = a3 ^ all ^ xt(a3 ^ a0);
      }
      for (int i = 0; i < 16; ++i) s[i] = t[i] ^ rk[r][i];
    }
    memcpy(out, s, 16);
  }
};

// X <- X * H in GF(2^128) with the GCM bit order (SP 800-38D, algorithm 1)
void gf128_mul(uint8_t x[16], const uint8_t h[16]) {
  uint8_t z[16] = {0}, v[16];
  memcpy(v, h, 16);
  for (int i = 0; i < 128; ++i) {
    if (x[i / 8] & (0x80 >> (i % 8))) for (int j = 0; j < 16; ++j) z[j] ^= v[j];
    bool lsb = v[15] & 1;
    for (int j = 15; j > 0; --j) v[j] = (uint8_t)((v[j] >> 1) | (v[j - 1] << 7));
    v[0] >>= 1;
    if (lsb) v[0] ^= 0xE1;
  }
  memcpy(x, z, 16);
}

void ghash_update(uint8_t y[16], const uint8_t h[16], const uint8_t* data, size_t len) {
  for (size_t off = 0; off < len; off += 16) {
    size_t n = len - off < 16 ? len - off : 16;
    for (size_t j = 0; j < n; ++j) y[j] ^= data[off + j];
    gf128_mul(y, h);
  }
}

void gcm_crypt(const uint8_t key[32], const uint8_t iv[12], const uint8_t* aad, size_t aadlen, const uint8_t* in, size_t len,
               uint8_t* out, uint8_t tag[16], bool encrypt) {
  Aes256 aes(key);
  uint8_t h[16] = {0}, j0[16] = {0}, ctr[16], ks[16], y[16] = {0};
  aes.encrypt(h, h);
  memcpy(j0, iv, 12);
  j0[15] = 1;
  memcpy(ctr, j0, 16);
  ghash_update(y, h, aad, aadlen);
  if (!encrypt) ghash_update(y, h, in, len);
  for (size_t off = 0; off < len; off += 16) {
    for (int j = 15; j >= 12; --j) if (++ctr[j]) break;
    aes.encrypt(ctr, ks);
    size_t n = len - off < 16 ? len - off : 16;
    for (size_t j = 0; j < n; ++j) out[off + j] = in[off + j] ^ ks[j];
  }
  if (encrypt) ghash_update(y, h, out, len);
  uint8_t lens[16];
  uint64_t ab = (uint64_t)aadlen * 8, cb = (uint64_t)len * 8;
  for (int i = 0; i < 8; ++i) { lens[i] = (uint8_t)(ab >> (56 - 8 * i)); lens[8 + i] = (uint8_t)(cb >> (56 - 8 * i)); }
  ghash_update(y, h, lens, 16);
  aes.encrypt(j0, ks);
  for (int i = 0; i < 16; ++i) tag[i] = y[i] ^ ks[i];
}

}  // namespace

SX_EXPORT void sx_aes256_encrypt_block(const void* key32, const void* in16, void* out16) { Aes256((const uint8_t*)key32).encrypt((const uint8_t*)in16, (uint8_t*)out16); }

// 96-bit IV. ct has `len` bytes, tag 16.
SX_EXPORT void sx_aes256_gcm_encrypt(const void* key, const void* iv12, const void* aad, size_t aadlen, const void* pt, size_t len, void* ct, void* tag16) {
  gcm_crypt((const uint8_t*)key, (const uint8_t*)iv12, (const uint8_t*)aad, aadlen, (const uint8_t*)pt, len, (uint8_t*)ct, (uint8_t*)tag16, true);
}

// Returns 0 and writes the plaintext when the tag verifies; -1 (and zeroes `pt`) otherwise.
SX_EXPORT int sx_aes256_gcm_decrypt(const void* key, const void* iv12, const void* aad, size_t aadlen, const void* ct, size_t len, const void* tag16, void* pt) {
  uint8_t tag[16];
  gcm_crypt((const uint8_t*)key, (const uint8_t*)iv12, (const uint8_t*)aad, aadlen, (const uint8_t*)ct, len, (uint8_t*)pt, tag, false);
  uint8_t diff = 0;
  for (int i = 0; i < 16; ++i) diff |= tag[i] ^ ((const uint8_t*)tag16)[i];
  if (diff) { memset(pt, 0, len); return -1; }
  return 0;
}

// ------------------------------------------------------------------------------------------------ Ed25519 (RFC 8032)
namespace {

typedef unsigned __int128 u128;
struct Fe { uint64_t v[5]; };  // value = sum v[i] * 2^(51 i), limbs kept below ~2^52 between operations
const uint64_t M51 = (1ULL << 51) - 1;

Fe fe_from_u64(uint64_t x) { return Fe{{x & M51, x >> 51, 0, 0, 0}}; }
Fe fe_carry(Fe a) {
  for (int r = 0; r < 2; ++r) {
    for (int i = 0; i < 4; ++i) { a.v[i + 1] += a.v[i] >> 51; a.v[i] &= M51; }
    a.v[0] += 19 * (a.v[4] >> 51); a.v[4] &= M51;
  }
  return a;
}
Fe fe_add(const Fe& a, const Fe& b) { Fe r; for (int i = 0; i < 5; ++i) r.v[i] = a.v[i] + b.v[i]; return fe_carry(r); }
Fe fe_sub(const Fe& a, const Fe& b) {
  // add 4p (limbwise) so that no limb goes negative
  static const uint64_t P4[5] = {4 * (M51 - 18), 4 * M51, 4 * M51, 4 * M51, 4 * M51};
  Fe r; for (int i = 0; i < 5; ++i) r.v[i] = a.v[i] + P4[i] - b.v[i]; return fe_carry(r);
}
Fe fe_mul(const Fe& a, const Fe& b) {
  u128 t[5] = {0, 0, 0, 0, 0};
  for (int i = 0; i < 5; ++i) for (int j = 0; j < 5; ++j) {
    u128 p = (u128)a.v[i] * b.v[j];
    if (i + j >= 5) t[i + j - 5] += p * 19; else t[i + j] += p;
  }
  Fe r; u128 c = 0;
  for (int i = 0; i < 5; ++i) { t[i] += c; r.v[i] = (uint64_t)t[i] & M51; c = t[i] >> 51; }
  r.v[0] += (uint64_t)c * 19;
  return fe_carry(r);
}
Fe fe_sq(const Fe& a) { return fe_mul(a, a); }
// a^e for a little-endian exponent of `n` bytes
Fe fe_pow(const Fe& a, const uint8_t* e, int n) {
  Fe r = fe_from_u64(1);
  for (int i = n * 8 - 1; i >= 0; --i) { r = fe_sq(r); if ((e[i / 8] >> (i % 8)) & 1) r = fe_mul(r, a); }
  return r;
}
void fe_tobytes(const Fe& in, uint8_t out[32]) {
  Fe a = fe_carry(in);
  // conditional subtraction of p, twice is enough after a full carry
  for (int r = 0; r < 2; ++r) {
    uint64_t t[5]; t[0] = a.v[0] + 19;
    for (int i = 0; i < 4; ++i) { t[i + 1] = a.v[i + 1] + (t[i] >> 51); t[i] &= M51; }
    if (t[4] >> 51) { t[4] &= M51; memcpy(a.v, t, sizeof t); }  // a >= p: a - p = a + 19 - 2^255
  }
  uint8_t buf[40] = {0};
  for (int i = 0; i < 5; ++i) for (int b = 0; b < 51; ++b) if ((a.v[i] >> b) & 1) { int k = 51 * i + b; buf[k / 8] |= (uint8_t)(1 << (k % 8)); }
  memcpy(out, buf, 32);
}
Fe fe_frombytes(const uint8_t in[32]) {
  Fe r = {{0, 0, 0, 0, 0}};
  for (int k = 0; k < 255; ++k) if ((in[k / 8] >> (k % 8)) & 1) r.v[k / 51] |= 1ULL << (k % 51);
  return r;
}
bool fe_eq(const Fe& a, const Fe& b) { uint8_t x[32], y[32]; fe_tobytes(a, x); fe_tobytes(b, y); return memcmp(x, y, 32) == 0; }
bool fe_isneg(const Fe& a) { uint8_t x[32]; fe_tobytes(a, x); return x[0] & 1; }
Fe fe_neg(const Fe& a) { return fe_sub(fe_from_u64(0), a); }

struct EdConsts {
  Fe d, d2, sqrt_m1;
  uint8_t p_minus_2[32], p58[32];  // exponents p - 2 and (p - 5) / 8
  EdConsts() {
    memset(p_minus_2, 0xFF, 32); p_minus_2[0] = 0xEB; p_minus_2[31] = 0x7F;
    memset(p58, 0xFF, 32); p58[0] = 0xFD; p58[31] = 0x0F;  // (2^255 - 24) / 8 = 2^252 - 3
    Fe inv = fe_pow(fe_from_u64(121666), p_minus_2, 32);
    d = fe_mul(fe_neg(fe_from_u64(121665)), inv);
    d2 = fe_add(d, d);
    uint8_t e[32]; memset(e, 0xFF, 32); e[0] = 0xFB; e[31] = 0x1F;  // (p - 1) / 4 = 2^253 - 5
    sqrt_m1 = fe_pow(fe_from_u64(2), e, 32);
  }
};
const EdConsts& edc() { static EdConsts c; return c; }

struct Pt { Fe X, Y, Z, T; };
Pt pt_identity() { return Pt{fe_from_u64(0), fe_from_u64(1), fe_from_u64(1), fe_from_u64(0)}; }
Pt pt_add(const Pt& p, const Pt& q) {  // unified addition on -x^2 + y^2 = 1 + d x^2 y^2, extended coordinates
  Fe A = fe_mul(fe_sub(p.Y, p.X), fe_sub(q.Y, q.X)), B = fe_mul(fe_add(p.Y, p.X), fe_add(q.Y, q.X));
  Fe C = fe_mul(fe_mul(p.T, edc().d2), q.T), D = fe_mul(fe_add(p.Z, p.Z), q.Z);
  Fe E = fe_sub(B, A), F = fe_sub(D, C), G = fe_add(D, C), H = fe_add(B, A);
  return Pt{fe_mul(E, F), fe_mul(G, H), fe_mul(F, G), fe_mul(E, H)};
}
Pt pt_mul(const Pt& p, const uint8_t k[32]) {
  Pt r = pt_identity();
  for (int i = 255; i >= 0; --i) { r = pt_add(r, r); if ((k[i / 8] >> (i % 8)) & 1) r = pt_add(r, p); }
  return r;
}
void pt_encode(const Pt& p, uint8_t out[32]) {
  Fe zi = fe_pow(p.Z, edc().p_minus_2, 32), x = fe_mul(p.X, zi), y = fe_mul(p.Y, zi);
  fe_tobytes(y, out);
  if (fe_isneg(x)) out[31] |= 0x80;
}
bool pt_decode(const uint8_t in[32], Pt& out) {
  uint8_t yb[32]; memcpy(yb, in, 32); bool sign = yb[31] >> 7; yb[31] &= 0x7F;
  Fe y = fe_frombytes(yb), one = fe_from_u64(1), y2 = fe_sq(y);
  Fe u = fe_sub(y2, one), v = fe_add(fe_mul(edc().d, y2), one);
  Fe v3 = fe_mul(fe_sq(v), v), v7 = fe_mul(fe_sq(v3), v);
  Fe x = fe_mul(fe_mul(u, v3), fe_pow(fe_mul(u, v7), edc().p58, 32));
  Fe vx2 = fe_mul(v, fe_sq(x));
  if (!fe_eq(vx2, u)) { if (fe_eq(vx2, fe_neg(u))) x = fe_mul(x, edc().sqrt_m1); else return false; }
  if (fe_isneg(x) != sign) { if (fe_eq(x, fe_from_u64(0))) return false; x = fe_neg(x); }
  out = Pt{x, y, one, fe_mul(x, y)};
  return true;
}
const Pt& base_point() {
  static Pt B = [] { uint8_t b[32]; memset(b, 0x66, 32); b[0] = 0x58; Pt p; pt_decode(b, p); return p; }();
  return B;
}

// scalars modulo the group order L = 2^252 + 27742317777372353535851937790883648493, as 32 little-endian bytes
const uint8_t ORDER_L[32] = {0xed, 0xd3, 0xf5, 0x5c, 0x1a, 0x63, 0x12, 0x58, 0xd6, 0x9c, 0xf7, 0xa2, 0xde, 0xf9, 0xde, 0x14,
                             0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0x10};
bool ge_bytes(const uint8_t* a, const uint8_t* b, int n) { for (int i = n - 1; i >= 0; --i) if (a[i] != b[i]) return a[i] > b[i]; return true; }
// out = in (n bytes, little-endian) mod L by shift-and-subtract
void sc_reduce(const uint8_t* in, int n, uint8_t out[32]) {
  uint8_t r[33] = {0};
  for (int bit = n * 8 - 1; bit >= 0; --bit) {
    for (int i = 32; i > 0; --i) r[i] = (uint8_t)((r[i] << 1) | (r[i - 1] >> 7));
    r[0] = (uint8_t)((r[0] << 1) | ((in[bit / 8] >> (bit % 8)) & 1));
    uint8_t l33[33]; memcpy(l33, ORDER_L, 32); l33[32] = 0;
    if (ge_bytes(r, l33, 33)) { int borrow = 0; for (int i = 0; i < 33; ++i) { int d = r[i] - l33[i] - borrow; borrow = d < 0; r[i] = (uint8_t)(d + (borrow << 8)); } }
  }
  memcpy(out, r, 32);
}
// out = (a * b + c) mod L
void sc_muladd(const uint8_t a[32], const uint8_t b[32], const uint8_t c[32], uint8_t out[32]) {
  uint32_t t[65] = {0};
  for (int i = 0; i < 32; ++i) for (int j = 0; j < 32; ++j) t[i + j] += (uint32_t)a[i] * b[j];
  for (int i = 0; i < 32; ++i) t[i] += c[i];
  uint8_t wide[65];
  uint32_t carry = 0;
  for (int i = 0; i < 65; ++i) { uint32_t v = t[i] + carry; wide[i] = (uint8_t)v; carry = v >> 8; }
  sc_reduce(wide, 65, out);
}

void ed_expand(const uint8_t seed[32], uint8_t a[32], uint8_t prefix[32]) {
  uint8_t h[64]; sha512(seed, 32, h);
  memcpy(a, h, 32); a[0] &= 248; a[31] &= 127; a[31] |= 64;
  memcpy(prefix, h + 32, 32);
}

}  // namespace

SX_EXPORT void sx_ed25519_public_key(const void* seed32, void* pub32) {
  uint8_t a[32], prefix[32]; ed_expand((const uint8_t*)seed32, a, prefix);
  pt_encode(pt_mul(base_point(), a), (uint8_t*)pub32);
}

SX_EXPORT void sx_ed25519_sign(const void* seed32, const void* msg, size_t len, void* sig64) {
  uint8_t a[32], prefix[32], A[32], r[32], k[32], h[64];
  ed_expand((const uint8_t*)seed32, a, prefix);
  pt_encode(pt_mul(base_point(), a), A);
  std::vector<uint8_t> buf(prefix, prefix + 32);
  buf.insert(buf.end(), (const uint8_t*)msg, (const uint8_t*)msg + len);
  sha512(buf.data(), buf.size(), h); sc_reduce(h, 64, r);
  uint8_t* sig = (uint8_t*)sig64;
  pt_encode(pt_mul(base_point(), r), sig);
  buf.assign(sig, sig + 32); buf.insert(buf.end(), A, A + 32);
  buf.insert(buf.end(), (const uint8_t*)msg, (const uint8_t*)msg + len);
  sha512(buf.data(), buf.size(), h); sc_reduce(h, 64, k);
  sc_muladd(k, a, r, sig + 32);
}

// 1 = valid, 0 = invalid
SX_EXPORT int sx_ed25519_verify(const void* pub32, const void* msg, size_t len, const void* sig64) {
  const uint8_t* sig = (const uint8_t*)sig64;
  if (ge_bytes(sig + 32, ORDER_L, 32)) return 0;  // S must be below L
  Pt A;
  if (!pt_decode((const uint8_t*)pub32, A)) return 0;
  uint8_t h[64], k[32], enc[32];
  std::vector<uint8_t> buf(sig, sig + 32);
  buf.insert(buf.end(), (const uint8_t*)pub32, (const uint8_t*)pub32 + 32);
  buf.insert(buf.end(), (const uint8_t*)msg, (const uint8_t*)msg + len);
  sha512(buf.data(), buf.size(), h); sc_reduce(h, 64, k);
  Pt negA{fe_neg(A.X), A.Y, A.Z, fe_neg(A.T)};
  pt_encode(pt_add(pt_mul(base_point(), sig + 32), pt_mul(negA, k)), enc);  // S B - k A must equal R
  return memcmp(enc, sig, 32) == 0;
}

// ------------------------------------------------------------------------------------------------ Schnorr proof of knowledge
// Non-interactive proof (Fiat-Shamir) that the prover knows x with P = x B on the Ed25519 group: R = k B,
// c = SHA-512(R || P || context) mod L, s = k + c x mod L; the proof is R || s. The nonce k is derived from the secret and
// the context (deterministic, never reused across contexts). Reference counterpart: drivers/zk/zk_proof.c.
namespace {
void schnorr_challenge(const uint8_t R[32], const uint8_t P[32], const uint8_t* ctx, size_t len, uint8_t c[32]) {
  std::vector<uint8_t> buf(R, R + 32);
  buf.insert(buf.end(), P, P + 32);
  buf.insert(buf.end(), ctx, ctx + len);
  uint8_t h[64];
  sha512(buf.data(), buf.size(), h);
  sc_reduce(h, 64, c);
}
}  // namespace

// secret: any 32 bytes (reduced mod L). Writes the public point P = x B.
SX_EXPORT void sx_schnorr_public(const void* secret32, void* pub32) {
  uint8_t x[32];
  sc_reduce((const uint8_t*)secret32, 32, x);
  pt_encode(pt_mul(base_point(), x), (uint8_t*)pub32);
}

SX_EXPORT void sx_schnorr_prove(const void* secret32, const void* context, size_t len, void* proof64) {
  uint8_t x[32], P[32], k[32], c[32], h[64];
  sc_reduce((const uint8_t*)secret32, 32, x);
  pt_encode(pt_mul(base_point(), x), P);
  std::vector<uint8_t> buf((const uint8_t*)secret32, (const uint8_t*)secret32 + 32);
  buf.insert(buf.end(), (const uint8_t*)context, (const uint8_t*)context + len);
  const char* tag = "sneppx-schnorr-nonce";
  buf.insert(buf.end(), tag, tag + 20);
  sha512(buf.data(), buf.size(), h);
  sc_reduce(h, 64, k);
  uint8_t* out = (uint8_t*)proof64;
  pt_encode(pt_mul(base_point(), k), out);
  schnorr_challenge(out, P, (const uint8_t*)context, len, c);
  sc_muladd(c, x, k, out + 32);
}

// 1 = the proof shows knowledge of the discrete logarithm of `pub32` for this context
SX_EXPORT int sx_schnorr_verify(const void* pub32, const void* context, size_t len, const void* proof64) {
  const uint8_t* pr = (const uint8_t*)proof64;
  if (ge_bytes(pr + 32, ORDER_L, 32)) return 0;
  Pt P;
  if (!pt_decode((const uint8_t*)pub32, P)) return 0;
  uint8_t c[32], enc[32];
  schnorr_challenge(pr, (const uint8_t*)pub32, (const uint8_t*)context, len, c);
  Pt negP{fe_neg(P.X), P.Y, P.Z, fe_neg(P.T)};
  pt_encode(pt_add(pt_mul(base_point(), pr + 32), pt_mul(negP, c)), enc);  // s B - c P must equal R
  return memcmp(enc, pr, 32) == 0;
}

// ------------------------------------------------------------------------------------------------ Argon2id (RFC 9106)
// Memory-hard password hashing, version 0x13, type id (data-independent addressing in the first half of the first
// pass, data-dependent afterwards). Lanes are filled one after another inside a slice (no threads).
namespace {

typedef uint64_t A2Block[128];

void a2_le32(std::vector<uint8_t>& v, uint32_t x) { for (int i = 0; i < 4; ++i) v.push_back((uint8_t)(x >> (8 * i))); }

// variable-length hash H' of RFC 9106 section 3.3
void a2_hprime(const uint8_t* in, size_t inlen, uint8_t* out, uint32_t T) {
  std::vector<uint8_t> buf;
  a2_le32(buf, T);
  buf.insert(buf.end(), in, in + inlen);
  if (T <= 64) { blake2b(buf.data(), buf.size(), nullptr, 0, out, T); return; }
  uint8_t v[64];
  blake2b(buf.data(), buf.size(), nullptr, 0, v, 64);
  const uint32_t r = (T + 31) / 32 - 2;
  memcpy(out, v, 32);
  for (uint32_t i = 1; i < r; ++i) { uint8_t nx[64]; blake2b(v, 64, nullptr, 0, nx, 64); memcpy(v, nx, 64); memcpy(out + 32 * i, v, 32); }
  blake2b(v, 64, nullptr, 0, out + 32 * r, T - 32 * r);
}

inline void a2_gb(uint64_t& a, uint64_t& b, uint64_t& c, uint64_t& d) {
  auto mix = [](uint64_t x, uint64_t y) { return x + y + 2 * (uint64_t)(uint32_t)x * (uint64_t)(uint32_t)y; };
  a = mix(a, b); d = rotr64(d ^ a, 32); c = mix(c, d); b = rotr64(b ^ c, 24);
  a = mix(a, b); d = rotr64(d ^ a, 16); c = mix(c, d); b = rotr64(b ^ c, 63);
}
inline void a2_p(uint64_t* v[16]) {
  a2_gb(*v[0], *v[4], *v[8], *v[12]); a2_gb(*v[1], *v[5], *v[9], *v[13]); a2_gb(*v[2], *v[6], *v[10], *v[14]); a2_gb(*v[3], *v[7], *v[11], *v[15]);
  a2_gb(*v[0], *v[5], *v[10], *v[15]); a2_gb(*v[1], *v[6], *v[11], *v[12]); a2_gb(*v[2], *v[7], *v[8], *v[13]); a2_gb(*v[3], *v[4], *v[9], *v[14]);
}
// out = G(x, y) (xor_into: out ^= G(x, y), the second and later passes)
void a2_g(const A2Block x, const A2Block y, A2Block out, bool xor_into) {
  A2Block r, z;
  for (int i = 0; i < 128; ++i) z[i] = r[i] = x[i] ^ y[i];
  for (int row = 0; row < 8; ++row) { uint64_t* v[16]; for (int i = 0; i < 16; ++i) v[i] = &z[16 * row + i]; a2_p(v); }
  for (int col = 0; col < 8; ++col) { uint64_t* v[16]; for (int i = 0; i < 8; ++i) { v[2 * i] = &z[16 * i + 2 * col]; v[2 * i + 1] = &z[16 * i + 2 * col + 1]; } a2_p(v); }
  for (int i = 0; i < 128; ++i) out[i] = (xor_into ? out[i] : 0) ^ z[i] ^ r[i];
}

}  // namespace

// m_kib: memory in KiB (>= 8 * lanes). Returns 0, or -1 on bad parameters.
SX_EXPORT int sx_argon2id(const void* pwd, size_t pwdlen, const void* salt, size_t saltlen, const void* secret, size_t secretlen,
                          const void* ad, size_t adlen, uint32_t t_cost, uint32_t m_kib, uint32_t lanes, void* out, uint32_t outlen) {
  if (lanes < 1 || t_cost < 1 || outlen < 4 || m_kib < 8 * lanes || saltlen < 8) return -1;
  const uint32_t mprime = 4 * lanes * (m_kib / (4 * lanes)), q = mprime / lanes, seg = q / 4;
  std::vector<uint8_t> h0in;
  a2_le32(h0in, lanes); a2_le32(h0in, outlen); a2_le32(h0in, m_kib); a2_le32(h0in, t_cost); a2_le32(h0in, 0x13); a2_le32(h0in, 2);
  auto field = [&](const void* p, size_t n) { a2_le32(h0in, (uint32_t)n); h0in.insert(h0in.end(), (const uint8_t*)p, (const uint8_t*)p + n); };
  field(pwd, pwdlen); field(salt, saltlen); field(secret, secretlen); field(ad, adlen);
  uint8_t h0[72];
  blake2b(h0in.data(), h0in.size(), nullptr, 0, h0, 64);
  std::vector<uint64_t> mem((size_t)mprime * 128);
  auto B = [&](uint32_t lane, uint32_t col) { return &mem[((size_t)lane * q + col) * 128]; };
  for (uint32_t l = 0; l < lanes; ++l)
    for (uint32_t c = 0; c < 2; ++c) {
      for (int i = 0; i < 4; ++i) { h0[64 + i] = (uint8_t)(c >> (8 * i)); h0[68 + i] = (uint8_t)(l >> (8 * i)); }
      a2_hprime(h0, 72, (uint8_t*)B(l, c), 1024);
    }
  A2Block zero = {0}, input, addr;
  for (uint32_t pass = 0; pass < t_cost; ++pass)
    for (uint32_t s = 0; s < 4; ++s)
      for (uint32_t l = 0; l < lanes; ++l) {
        const bool indep = pass == 0 && s < 2;
        uint32_t start = (pass == 0 && s == 0) ? 2 : 0;
        auto next_addresses = [&] { ++input[6]; A2Block tmp; a2_g(zero, input, tmp, false); a2_g(zero, tmp, addr, false); };
        if (indep) {
          memset(input, 0, sizeof input);
          input[0] = pass; input[1] = l; input[2] = s; input[3] = mprime; input[4] = t_cost; input[5] = 2;
          if (start) next_addresses();
        }
        for (uint32_t idx = start; idx < seg; ++idx) {
          const uint32_t j = s * seg + idx, prev = j ? j - 1 : q - 1;
          uint64_t rnd;
          if (indep) { if (idx % 128 == 0) next_addresses(); rnd = addr[idx % 128]; }
          else rnd = B(l, prev)[0];
          const uint32_t j1 = (uint32_t)rnd, j2 = (uint32_t)(rnd >> 32);
          const uint32_t ref_lane = (pass == 0 && s == 0) ? l : j2 % lanes;
          const bool same = ref_lane == l;
          uint32_t area;
          if (pass == 0) area = s == 0 ? idx - 1 : (same ? s * seg + idx - 1 : s * seg - (idx == 0 ? 1 : 0));
          else area = same ? q - seg + idx - 1 : q - seg - (idx == 0 ? 1 : 0);
          const uint64_t x = ((uint64_t)j1 * j1) >> 32, y = ((uint64_t)area * x) >> 32;
          const uint32_t zz = area - 1 - (uint32_t)y;
          const uint32_t first = (pass != 0 && s != 3) ? (s + 1) * seg : 0;
          const uint32_t ref = (first + zz) % q;
          a2_g(B(l, prev), B(ref_lane, ref), B(l, j), pass > 0);
        }
      }
  A2Block fin;
  memcpy(fin, B(0, q - 1), sizeof fin);
  for (uint32_t l = 1; l < lanes; ++l) for (int i = 0; i < 128; ++i) fin[i] ^= B(l, q - 1)[i];
  a2_hprime((const uint8_t*)fin, 1024, (uint8_t*)out, outlen);
  return 0;
}

// ------------------------------------------------------------------------------------------------ BLAKE3
// Hash and keyed-hash modes with extendable output: 1024-byte chunks of 64-byte blocks, a binary tree of chaining
// values merged with a stack, and the root node re-compressed per 64-byte output block.
namespace {

const uint32_t B3_IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
const int B3_PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum { B3_CHUNK_START = 1, B3_CHUNK_END = 2, B3_PARENT = 4, B3_ROOT = 8, B3_KEYED = 16 };

inline uint32_t rotr32(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

void b3_compress(const uint32_t cv[8], const uint32_t block[16], uint64_t counter, uint32_t block_len, uint32_t flags, uint32_t out[16]) {
  uint32_t s[16] = {cv[0], cv[1], cv[2], cv[3], cv[4], cv[5], cv[6], cv[7], B3_IV[0], B3_IV[1], B3_IV[2], B3_IV[3],
                    (uint32_t)counter, (uint32_t)(counter >> 32), block_len, flags};
  uint32_t m[16];
  memcpy(m, block, sizeof m);
  auto g = [&](int a, int b, int c, int d, uint32_t mx, uint32_t my) {
    s[a] = s[a] + s[b] + mx; s[d] = rotr32(s[d] ^ s[a], 16); s[c] = s[c] + s[d]; s[b] = rotr32(s[b] ^ s[c], 12);
    s[a] = s[a] + s[b] + my; s[d] = rotr32(s[d] ^ s[a], 8); s[c] = s[c] + s[d]; s[b] = rotr32(s[b] ^ s[c], 7);
  };
  for (int r = 0; r < 7; ++r) {
    g(0, 4, 8, 12, m[0], m[1]); g(1, 5, 9, 13, m[2], m[3]); g(2, 6, 10, 14, m[4], m[5]); g(3, 7, 11, 15, m[6], m[7]);
    g(0, 5, 10, 15, m[8], m[9]); g(1, 6, 11, 12, m[10], m[11]); g(2, 7, 8, 13, m[12], m[13]); g(3, 4, 9, 14, m[14], m[15]);
    uint32_t t[16];
    for (int i = 0; i < 16; ++i) t[i] = m[B3_PERM[i]];
    memcpy(m, t, sizeof m);
  }
  for (int i = 0; i < 8; ++i) { out[i] = s[i] ^ s[i + 8]; out[i + 8] = s[i + 8] ^ cv[i]; }
}

struct B3Output { uint32_t cv[8], block[16]; uint64_t counter; uint32_t block_len, flags; };

void b3_words(const uint8_t* p, size_t n, uint32_t w[16]) {
  uint8_t buf[64] = {0};
  memcpy(buf, p, n);
  for (int i = 0; i < 16; ++i) w[i] = (uint32_t)buf[4 * i] | (uint32_t)buf[4 * i + 1] << 8 | (uint32_t)buf[4 * i + 2] << 16 | (uint32_t)buf[4 * i + 3] << 24;
}

// the last block of a chunk is returned uncompressed (it may turn out to be the root)
B3Output b3_chunk(const uint32_t key[8], const uint8_t* p, size_t len, uint64_t index, uint32_t base) {
  B3Output o;
  memcpy(o.cv, key, 32);
  const size_t nb = len ? (len + 63) / 64 : 1;
  for (size_t b = 0; b < nb; ++b) {
    const size_t off = 64 * b, bl = b + 1 < nb ? 64 : len - off;
    uint32_t w[16];
    b3_words(p + off, bl, w);
    const uint32_t fl = base | (b == 0 ? B3_CHUNK_START : 0) | (b + 1 == nb ? B3_CHUNK_END : 0);
    if (b + 1 < nb) { uint32_t out[16]; b3_compress(o.cv, w, index, 64, fl, out); memcpy(o.cv, out, 32); }
    else { memcpy(o.block, w, 64); o.counter = index; o.block_len = (uint32_t)bl; o.flags = fl; }
  }
  return o;
}

void b3_cv_of(const B3Output& o, uint32_t cv[8]) {
  uint32_t out[16];
  b3_compress(o.cv, o.block, o.counter, o.block_len, o.flags, out);
  memcpy(cv, out, 32);
}

B3Output b3_parent(const uint32_t left[8], const uint32_t right[8], const uint32_t key[8], uint32_t base) {
  B3Output o;
  memcpy(o.cv, key, 32);
  memcpy(o.block, left, 32);
  memcpy(o.block + 8, right, 32);
  o.counter = 0; o.block_len = 64; o.flags = base | B3_PARENT;
  return o;
}

}  // namespace

// key32 == nullptr: plain hash; otherwise the keyed mode. Any output length (extendable output).
SX_EXPORT void sx_blake3(const void* msg, size_t len, const void* key32, void* out, size_t outlen) {
  uint32_t key[8];
  uint32_t base = 0;
  if (key32) { uint32_t w[16]; b3_words((const uint8_t*)key32, 32, w); memcpy(key, w, 32); base = B3_KEYED; }
  else memcpy(key, B3_IV, 32);
  const uint8_t* p = (const uint8_t*)msg;
  const size_t chunks = len ? (len + 1023) / 1024 : 1;
  std::vector<std::vector<uint32_t>> stack;
  for (size_t c = 0; c + 1 < chunks; ++c) {
    uint32_t cv[8];
    b3_cv_of(b3_chunk(key, p + 1024 * c, 1024, c, base), cv);
    size_t total = c + 1;   // chunks completed so far: merge one level per trailing zero bit
    while ((total & 1) == 0) {
      uint32_t merged[8];
      b3_cv_of(b3_parent(stack.back().data(), cv, key, base), merged);
      stack.pop_back();
      memcpy(cv, merged, 32);
      total >>= 1;
    }
    stack.emplace_back(cv, cv + 8);
  }
  B3Output o = b3_chunk(key, p + 1024 * (chunks - 1), len - 1024 * (chunks - 1), chunks - 1, base);
  while (!stack.empty()) {
    uint32_t cv[8];
    b3_cv_of(o, cv);
    o = b3_parent(stack.back().data(), cv, key, base);
    stack.pop_back();
  }
  uint8_t* dst = (uint8_t*)out;
  for (uint64_t blk = 0; outlen; ++blk) {
    uint32_t w[16];
    b3_compress(o.cv, o.block, blk, o.block_len, o.flags | B3_ROOT, w);
    uint8_t bytes[64];
    for (int i = 0; i < 16; ++i) for (int j = 0; j < 4; ++j) bytes[4 * i + j] = (uint8_t)(w[i] >> (8 * j));
    const size_t n = outlen < 64 ? outlen : 64;
    memcpy(dst, bytes, n);
    dst += n; outlen -= n;
  }
}
