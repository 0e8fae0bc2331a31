// Stateless hash-based signatures: SLH-DSA (FIPS 205, the standardised form of SPHINCS+) with SHAKE-256, parameter
// sets 128f (fast signing, 17 088-byte signatures) and 128s (small, 7 856 bytes).
//
// Reference counterpart: security/crypto/post_quantum (SPHINCS+). Written from FIPS 205: WOTS+ one-time signatures
// (w = 16), XMSS trees stacked into a hypertree, a FORS few-time signature of the message digest, and the 32-byte
// address structure that separates every hash call. No independent implementation of this scheme is available to the
// tests, so they check the scheme's own properties (sizes, determinism, acceptance, rejection of any changed byte,
// message, context or key); byte-level agreement with other implementations has not been checked.
#include <cstdint>
#include <cstring>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

extern "C" void sx_shake256(const void* msg, size_t len, void* out, size_t outlen);

namespace {

constexpr int NB = 16;                 // n: bytes per hash value (both 128-bit parameter sets)
constexpr int LEN1 = 2 * NB, LEN2 = 3, LEN = LEN1 + LEN2, W = 16;
enum AdrsType { WOTS_HASH = 0, WOTS_PK = 1, TREE = 2, FORS_TREE = 3, FORS_ROOTS = 4, WOTS_PRF = 5, FORS_PRF = 6 };

struct Params { int h, d, hp, a, k, m; };
bool params_for(int variant, Params& p) {
  if (variant == 0) p = {66, 22, 3, 6, 33, 34};         // 128f
  else if (variant == 1) p = {63, 7, 9, 12, 14, 30};    // 128s
  else return false;
  return true;
}
inline int sig_len(const Params& p) { return NB * (1 + p.k * (1 + p.a) + p.h + p.d * LEN); }

struct Adrs {
  uint8_t b[32];
  Adrs() { memset(b, 0, 32); }
  static void put32(uint8_t* p, uint32_t v) { p[0] = (uint8_t)(v >> 24); p[1] = (uint8_t)(v >> 16); p[2] = (uint8_t)(v >> 8); p[3] = (uint8_t)v; }
  static uint32_t get32(const uint8_t* p) { return ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | p[3]; }
  void layer(uint32_t v) { put32(b, v); }
  void tree(uint64_t v) { put32(b + 4, 0); put32(b + 8, (uint32_t)(v >> 32)); put32(b + 12, (uint32_t)v); }
  void type_and_clear(uint32_t t) { put32(b + 16, t); memset(b + 20, 0, 12); }
  void keypair(uint32_t v) { put32(b + 20, v); }
  uint32_t keypair() const { return get32(b + 20); }
  void chain(uint32_t v) { put32(b + 24, v); }        // also the tree height of TREE / FORS_TREE addresses
  void height(uint32_t v) { put32(b + 24, v); }
  void hash(uint32_t v) { put32(b + 28, v); }         // also the tree index
  void index(uint32_t v) { put32(b + 28, v); }
  uint32_t index() const { return get32(b + 28); }
};

struct Ctx { const uint8_t* pk_seed; const uint8_t* sk_seed; Params P; };

// F, H and T_l: SHAKE256(PK.seed || ADRS || M) truncated to n bytes
void thash(const Ctx& c, const Adrs& a, const uint8_t* in, size_t inlen, uint8_t* out) {
  uint8_t stack[NB + 32 + LEN * NB];
  memcpy(stack, c.pk_seed, NB); memcpy(stack + NB, a.b, 32); memcpy(stack + NB + 32, in, inlen);
  sx_shake256(stack, NB + 32 + inlen, out, NB);
}
void prf(const Ctx& c, const Adrs& a, uint8_t* out) {
  uint8_t stack[NB + 32 + NB];
  memcpy(stack, c.pk_seed, NB); memcpy(stack + NB, a.b, 32); memcpy(stack + NB + 32, c.sk_seed, NB);
  sx_shake256(stack, sizeof(stack), out, NB);
}

void base_2b(const uint8_t* x, int b, int out_len, uint32_t* out) {
  uint32_t total = 0; int bits = 0, in = 0;
  for (int i = 0; i < out_len; ++i) {
    while (bits < b) { total = (total << 8) | x[in++]; bits += 8; }
    bits -= b;
    out[i] = (total >> bits) & ((1u << b) - 1);
  }
}

// ----------------------------------------------------------------------------------------------- WOTS+
void chain(const Ctx& c, const uint8_t* x, int start, int steps, Adrs& a, uint8_t* out) {
  memcpy(out, x, NB);
  for (int j = start; j < start + steps; ++j) { a.hash((uint32_t)j); thash(c, a, out, NB, out); }
}
void wots_digits(const uint8_t* msg, uint32_t* d) {
  base_2b(msg, 4, LEN1, d);
  uint32_t csum = 0;
  for (int i = 0; i < LEN1; ++i) csum += W - 1 - d[i];
  csum <<= 4;                                       // (8 - (len2 * lg_w) % 8) % 8
  const uint8_t cs[2] = {(uint8_t)(csum >> 8), (uint8_t)csum};
  base_2b(cs, 4, LEN2, d + LEN1);
}
void wots_pk_gen(const Ctx& c, Adrs& a, uint8_t* pk) {
  Adrs sk_a = a;
  sk_a.type_and_clear(WOTS_PRF); sk_a.keypair(a.keypair());
  uint8_t tmp[LEN * NB], sk[NB];
  for (int i = 0; i < LEN; ++i) {
    sk_a.chain((uint32_t)i); prf(c, sk_a, sk);
    a.chain((uint32_t)i); chain(c, sk, 0, W - 1, a, tmp + i * NB);
  }
  Adrs pk_a = a;
  pk_a.type_and_clear(WOTS_PK); pk_a.keypair(a.keypair());
  thash(c, pk_a, tmp, sizeof(tmp), pk);
}
void wots_sign(const Ctx& c, const uint8_t* msg, Adrs& a, uint8_t* sig) {
  uint32_t d[LEN];
  wots_digits(msg, d);
  Adrs sk_a = a;
  sk_a.type_and_clear(WOTS_PRF); sk_a.keypair(a.keypair());
  uint8_t sk[NB];
  for (int i = 0; i < LEN; ++i) {
    sk_a.chain((uint32_t)i); prf(c, sk_a, sk);
    a.chain((uint32_t)i); chain(c, sk, 0, (int)d[i], a, sig + i * NB);
  }
}
void wots_pk_from_sig(const Ctx& c, const uint8_t* sig, const uint8_t* msg, Adrs& a, uint8_t* pk) {
  uint32_t d[LEN];
  wots_digits(msg, d);
  uint8_t tmp[LEN * NB];
  for (int i = 0; i < LEN; ++i) { a.chain((uint32_t)i); chain(c, sig + i * NB, (int)d[i], W - 1 - (int)d[i], a, tmp + i * NB); }
  Adrs pk_a = a;
  pk_a.type_and_clear(WOTS_PK); pk_a.keypair(a.keypair());
  thash(c, pk_a, tmp, sizeof(tmp), pk);
}

// ----------------------------------------------------------------------------------------------- XMSS / hypertree
void xmss_node(const Ctx& c, uint32_t i, int z, Adrs& a, uint8_t* node) {
  if (z == 0) { a.type_and_clear(WOTS_HASH); a.keypair(i); wots_pk_gen(c, a, node); return; }
  uint8_t lr[2 * NB];
  xmss_node(c, 2 * i, z - 1, a, lr);
  xmss_node(c, 2 * i + 1, z - 1, a, lr + NB);
  a.type_and_clear(TREE); a.height((uint32_t)z); a.index(i);
  thash(c, a, lr, 2 * NB, node);
}
void xmss_sign(const Ctx& c, const uint8_t* msg, uint32_t idx, Adrs& a, uint8_t* sig) {
  for (int j = 0; j < c.P.hp; ++j) xmss_node(c, (idx >> j) ^ 1, j, a, sig + (LEN + j) * NB);
  a.type_and_clear(WOTS_HASH); a.keypair(idx);
  wots_sign(c, msg, a, sig);
}
void xmss_pk_from_sig(const Ctx& c, uint32_t idx, const uint8_t* sig, const uint8_t* msg, Adrs& a, uint8_t* root) {
  a.type_and_clear(WOTS_HASH); a.keypair(idx);
  uint8_t node[2 * NB], cat[2 * NB];
  wots_pk_from_sig(c, sig, msg, a, node);
  a.type_and_clear(TREE); a.index(idx);
  for (int k = 0; k < c.P.hp; ++k) {
    const uint8_t* auth = sig + (LEN + k) * NB;
    a.height((uint32_t)(k + 1));
    if (((idx >> k) & 1) == 0) { a.index(a.index() / 2); memcpy(cat, node, NB); memcpy(cat + NB, auth, NB); }
    else { a.index((a.index() - 1) / 2); memcpy(cat, auth, NB); memcpy(cat + NB, node, NB); }
    thash(c, a, cat, 2 * NB, node);
  }
  memcpy(root, node, NB);
}
void ht_sign(const Ctx& c, const uint8_t* msg, uint64_t idx_tree, uint32_t idx_leaf, uint8_t* sig) {
  const int xlen = (LEN + c.P.hp) * NB;
  uint8_t root[NB];
  memcpy(root, msg, NB);
  for (int j = 0; j < c.P.d; ++j) {
    Adrs a; a.layer((uint32_t)j); a.tree(idx_tree);
    xmss_sign(c, root, idx_leaf, a, sig + j * xlen);
    if (j < c.P.d - 1) {
      xmss_pk_from_sig(c, idx_leaf, sig + j * xlen, root, a, root);
      idx_leaf = (uint32_t)(idx_tree & ((1u << c.P.hp) - 1));
      idx_tree >>= c.P.hp;
    }
  }
}
bool ht_verify(const Ctx& c, const uint8_t* msg, const uint8_t* sig, uint64_t idx_tree, uint32_t idx_leaf, const uint8_t* pk_root) {
  const int xlen = (LEN + c.P.hp) * NB;
  uint8_t node[NB];
  memcpy(node, msg, NB);
  for (int j = 0; j < c.P.d; ++j) {
    Adrs a; a.layer((uint32_t)j); a.tree(idx_tree);
    xmss_pk_from_sig(c, idx_leaf, sig + j * xlen, node, a, node);
    idx_leaf = (uint32_t)(idx_tree & ((1u << c.P.hp) - 1));
    idx_tree >>= c.P.hp;
  }
  uint8_t diff = 0;
  for (int i = 0; i < NB; ++i) diff |= (uint8_t)(node[i] ^ pk_root[i]);
  return diff == 0;
}

// ----------------------------------------------------------------------------------------------- FORS
void fors_sk(const Ctx& c, const Adrs& a, uint32_t idx, uint8_t* out) {
  Adrs s = a;
  s.type_and_clear(FORS_PRF); s.keypair(a.keypair()); s.index(idx);
  prf(c, s, out);
}
void fors_node(const Ctx& c, uint32_t i, int z, Adrs& a, uint8_t* node) {
  if (z == 0) {
    uint8_t sk[NB];
    fors_sk(c, a, i, sk);
    a.height(0); a.index(i);
    thash(c, a, sk, NB, node);
    return;
  }
  uint8_t lr[2 * NB];
  fors_node(c, 2 * i, z - 1, a, lr);
  fors_node(c, 2 * i + 1, z - 1, a, lr + NB);
  a.height((uint32_t)z); a.index(i);
  thash(c, a, lr, 2 * NB, node);
}
void fors_sign(const Ctx& c, const uint8_t* md, Adrs& a, uint8_t* sig) {
  uint32_t idx[40];
  base_2b(md, c.P.a, c.P.k, idx);
  for (int i = 0; i < c.P.k; ++i) {
    uint8_t* s = sig + (size_t)i * (1 + c.P.a) * NB;
    fors_sk(c, a, ((uint32_t)i << c.P.a) + idx[i], s);
    for (int j = 0; j < c.P.a; ++j)
      fors_node(c, ((uint32_t)i << (c.P.a - j)) + ((idx[i] >> j) ^ 1), j, a, s + (1 + j) * NB);
  }
}
void fors_pk_from_sig(const Ctx& c, const uint8_t* sig, const uint8_t* md, Adrs& a, uint8_t* pk) {
  uint32_t idx[40];
  base_2b(md, c.P.a, c.P.k, idx);
  uint8_t roots[40 * NB], node[NB], cat[2 * NB];
  for (int i = 0; i < c.P.k; ++i) {
    const uint8_t* s = sig + (size_t)i * (1 + c.P.a) * NB;
    a.height(0); a.index(((uint32_t)i << c.P.a) + idx[i]);
    thash(c, a, s, NB, node);
    for (int j = 0; j < c.P.a; ++j) {
      const uint8_t* auth = s + (1 + j) * NB;
      a.height((uint32_t)(j + 1));
      if (((idx[i] >> j) & 1) == 0) { a.index(a.index() / 2); memcpy(cat, node, NB); memcpy(cat + NB, auth, NB); }
      else { a.index((a.index() - 1) / 2); memcpy(cat, auth, NB); memcpy(cat + NB, node, NB); }
      thash(c, a, cat, 2 * NB, node);
    }
    memcpy(roots + i * NB, node, NB);
  }
  Adrs r = a;
  r.type_and_clear(FORS_ROOTS); r.keypair(a.keypair());
  uint8_t buf[NB + 32 + 40 * NB];
  memcpy(buf, c.pk_seed, NB); memcpy(buf + NB, r.b, 32); memcpy(buf + NB + 32, roots, (size_t)c.P.k * NB);
  sx_shake256(buf, NB + 32 + (size_t)c.P.k * NB, pk, NB);
}

// digest -> (FORS message, tree index, leaf index)
void split_digest(const Params& P, const uint8_t* digest, const uint8_t** md, uint64_t* idx_tree, uint32_t* idx_leaf) {
  const int md_len = (P.k * P.a + 7) / 8, tree_len = (P.h - P.h / P.d + 7) / 8, leaf_len = (P.h / P.d + 7) / 8;
  *md = digest;
  uint64_t t = 0;
  for (int i = 0; i < tree_len; ++i) t = (t << 8) | digest[md_len + i];
  const int tree_bits = P.h - P.h / P.d;
  *idx_tree = tree_bits >= 64 ? t : t & ((1ULL << tree_bits) - 1);
  uint32_t l = 0;
  for (int i = 0; i < leaf_len; ++i) l = (l << 8) | digest[md_len + tree_len + i];
  *idx_leaf = l & ((1u << (P.h / P.d)) - 1);
}
std::vector<uint8_t> framed(const uint8_t* prefix, size_t plen, const uint8_t* ctx, size_t clen, const uint8_t* msg, size_t mlen) {
  std::vector<uint8_t> v(plen + 2 + clen + mlen);
  memcpy(v.data(), prefix, plen);
  v[plen] = 0; v[plen + 1] = (uint8_t)clen;
  if (clen) memcpy(v.data() + plen + 2, ctx, clen);
  if (mlen) memcpy(v.data() + plen + 2 + clen, msg, mlen);
  return v;
}

}  // namespace

SX_EXPORT int sx_slhdsa_sizes(int variant, int* pk, int* sk, int* sig) {
  Params P;
  if (!params_for(variant, P)) return -1;
  *pk = 2 * NB; *sk = 4 * NB; *sig = sig_len(P);
  return 0;
}

// Key pair from three 16-byte seeds (SK.seed, SK.prf, PK.seed): sk = seeds || root, pk = PK.seed || root.
SX_EXPORT int sx_slhdsa_keygen(int variant, const uint8_t* seeds48, uint8_t* pk, uint8_t* sk) {
  Ctx c;
  if (!params_for(variant, c.P)) return -1;
  memcpy(sk, seeds48, 3 * NB);
  c.sk_seed = sk; c.pk_seed = sk + 2 * NB;
  Adrs a; a.layer((uint32_t)(c.P.d - 1));
  xmss_node(c, 0, c.P.hp, a, sk + 3 * NB);
  memcpy(pk, sk + 2 * NB, 2 * NB);
  return 0;
}

// `addrnd`: 16 bytes of fresh randomness (hedged) or null (deterministic: PK.seed takes its place).
SX_EXPORT int sx_slhdsa_sign(int variant, const uint8_t* sk, const uint8_t* msg, size_t mlen, const uint8_t* ctx, size_t clen,
                             const uint8_t* addrnd, uint8_t* sig) {
  Ctx c;
  if (!params_for(variant, c.P) || clen > 255) return -1;
  c.sk_seed = sk; c.pk_seed = sk + 2 * NB;
  const uint8_t *sk_prf = sk + NB, *pk_root = sk + 3 * NB;
  uint8_t head[3 * NB];
  memcpy(head, sk_prf, NB); memcpy(head + NB, addrnd ? addrnd : c.pk_seed, NB);
  std::vector<uint8_t> in = framed(head, 2 * NB, ctx, clen, msg, mlen);
  sx_shake256(in.data(), in.size(), sig, NB);                                    // R
  memcpy(head, sig, NB); memcpy(head + NB, c.pk_seed, NB); memcpy(head + 2 * NB, pk_root, NB);
  in = framed(head, 3 * NB, ctx, clen, msg, mlen);
  uint8_t digest[64];
  sx_shake256(in.data(), in.size(), digest, (size_t)c.P.m);
  const uint8_t* md; uint64_t idx_tree; uint32_t idx_leaf;
  split_digest(c.P, digest, &md, &idx_tree, &idx_leaf);
  Adrs a; a.tree(idx_tree); a.type_and_clear(FORS_TREE); a.keypair(idx_leaf);
  uint8_t* sig_fors = sig + NB;
  fors_sign(c, md, a, sig_fors);
  uint8_t pk_fors[NB];
  fors_pk_from_sig(c, sig_fors, md, a, pk_fors);
  ht_sign(c, pk_fors, idx_tree, idx_leaf, sig_fors + (size_t)c.P.k * (1 + c.P.a) * NB);
  return 0;
}

SX_EXPORT int sx_slhdsa_verify(int variant, const uint8_t* pk, const uint8_t* msg, size_t mlen, const uint8_t* ctx, size_t clen,
                               const uint8_t* sig) {
  Ctx c;
  if (!params_for(variant, c.P) || clen > 255) return 0;
  c.pk_seed = pk; c.sk_seed = nullptr;
  uint8_t head[3 * NB];
  memcpy(head, sig, NB); memcpy(head + NB, pk, 2 * NB);
  std::vector<uint8_t> in = framed(head, 3 * NB, ctx, clen, msg, mlen);
  uint8_t digest[64];
  sx_shake256(in.data(), in.size(), digest, (size_t)c.P.m);
  const uint8_t* md; uint64_t idx_tree; uint32_t idx_leaf;
  split_digest(c.P, digest, &md, &idx_tree, &idx_leaf);
  Adrs a; a.tree(idx_tree); a.type_and_clear(FORS_TREE); a.keypair(idx_leaf);
  const uint8_t* sig_fors = sig + NB;
  uint8_t pk_fors[NB];
  fors_pk_from_sig(c, sig_fors, md, a, pk_fors);
  return ht_verify(c, pk_fors, sig_fors + (size_t)c.P.k * (1 + c.P.a) * NB, idx_tree, idx_leaf, pk + NB) ? 1 : 0;
}
