// Host memory management: chunked arena, slab cache with per-thread magazines, virtual-memory reserve / commit,
// object pool, tiered memory with migration, huge-page advice, and block-floating-point / sparse compression codecs.
//
// Reference counterparts: mm/arena/arena_alloc.c, mm/internal/slab_alloc.c, mm/internal/vmem.c, mm/pool/object_pool.c,
// mm/tiered/tiered_memory.c, mm/huge/hugepage_mgr.c, mm/internal/compress.c. Device memory is not managed here: GPU
// tensors live in PyTorch's caching allocator and the symmetric-memory pool; these allocators serve the host runtime
// (checkpoint staging, tokenizer, serving queues) and the codecs serve cold-tier storage of activations and KV blocks.
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#define SX_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------------------------------------------------------
// Arena: bump allocation out of chunks; reset keeps the first chunk and releases the rest.
// ---------------------------------------------------------------------------------------------------------------
struct Arena {
  struct Chunk { char* base; size_t cap, used; };
  std::vector<Chunk> chunks;
  size_t chunk_size, n_allocs = 0, peak = 0;
  std::mutex mu;

  explicit Arena(size_t cs) : chunk_size(std::max<size_t>(cs, 4096)) { grow(chunk_size); }
  ~Arena() { for (auto& c : chunks) std::free(c.base); }
  void grow(size_t need) {
    size_t cap = std::max(chunk_size, need);
    chunks.push_back({(char*)std::aligned_alloc(4096, round_up(cap, 4096)), round_up(cap, 4096), 0});
  }
  size_t used() const { size_t u = 0; for (auto& c : chunks) u += c.used; return u; }
  size_t capacity() const { size_t u = 0; for (auto& c : chunks) u += c.cap; return u; }
  void* alloc(size_t n, size_t align) {
    std::lock_guard<std::mutex> lk(mu);
    if (align == 0 || (align & (align - 1))) return nullptr;
    auto& c = chunks.back();
    size_t off = round_up((size_t)(uintptr_t)(c.base + c.used), align) - (size_t)(uintptr_t)c.base;
    if (off + n > c.cap) {
      grow(n + align);
      return alloc_in_new(n, align);
    }
    c.used = off + n; ++n_allocs; peak = std::max(peak, used());
    return c.base + off;
  }
  void* alloc_in_new(size_t n, size_t align) {
    auto& c = chunks.back();
    size_t off = round_up((size_t)(uintptr_t)c.base, align) - (size_t)(uintptr_t)c.base;
    c.used = off + n; ++n_allocs; peak = std::max(peak, used());
    return c.base + off;
  }
  void reset() {
    std::lock_guard<std::mutex> lk(mu);
    for (size_t i = 1; i < chunks.size(); ++i) std::free(chunks[i].base);
    chunks.resize(1); chunks[0].used = 0;
  }
};

// ---------------------------------------------------------------------------------------------------------------
// Slab cache: fixed-size objects carved out of slabs; empty slabs are returned by gc(). A magazine is a per-thread
// stack of free objects that is refilled from / flushed to the cache in batches, so the lock is taken once per batch.
// ---------------------------------------------------------------------------------------------------------------
struct SlabCache {
  struct Slab { char* base; int in_use; };
  size_t obj_size; int per_slab;
  std::vector<Slab> slabs;
  std::vector<void*> free_list;
  std::mutex mu;
  size_t n_alloc = 0, n_free = 0;

  SlabCache(size_t os, int ps) : obj_size(round_up(std::max<size_t>(os, 8), 8)), per_slab(std::max(ps, 1)) {}
  ~SlabCache() { for (auto& s : slabs) std::free(s.base); }
  int slab_of(void* p) {
    for (size_t i = 0; i < slabs.size(); ++i)
      if ((char*)p >= slabs[i].base && (char*)p < slabs[i].base + obj_size * per_slab) return (int)i;
    return -1;
  }
  void* alloc_locked() {
    if (free_list.empty()) {
      char* b = (char*)std::aligned_alloc(64, round_up(obj_size * per_slab, 64));
      slabs.push_back({b, 0});
      for (int i = per_slab - 1; i >= 0; --i) free_list.push_back(b + obj_size * i);
    }
    void* p = free_list.back(); free_list.pop_back();
    slabs[slab_of(p)].in_use++; ++n_alloc;
    return p;
  }
  int free_locked(void* p) {
    int s = slab_of(p);
    if (s < 0) return -1;
    slabs[s].in_use--; free_list.push_back(p); ++n_free;
    return 0;
  }
  int gc() {
    std::lock_guard<std::mutex> lk(mu);
    int released = 0;
    for (size_t i = 0; i < slabs.size();) {
      if (slabs[i].in_use == 0) {
        char* b = slabs[i].base; char* e = b + obj_size * per_slab;
        free_list.erase(std::remove_if(free_list.begin(), free_list.end(), [&](void* p) { return (char*)p >= b && (char*)p < e; }), free_list.end());
        std::free(b); slabs.erase(slabs.begin() + i); ++released;
      } else ++i;
    }
    return released;
  }
};

struct Magazine {
  SlabCache* cache; int cap; std::vector<void*> items;
};

// ---------------------------------------------------------------------------------------------------------------
// Object pool: bounded set of equally sized, zero-initialised objects handed out and taken back.
// ---------------------------------------------------------------------------------------------------------------
struct ObjPool {
  size_t obj_size; int capacity; std::vector<void*> free_objs, all; std::mutex mu;
};

// ---------------------------------------------------------------------------------------------------------------
// Tiered memory: tier 0 is the fastest; an allocation that does not fit its preferred tier falls to the next one.
// ---------------------------------------------------------------------------------------------------------------
struct Tiered {
  struct Block { size_t size; int tier; };
  std::vector<size_t> cap, used; std::vector<std::string> names;
  std::map<void*, Block> blocks; std::mutex mu;
};

}  // namespace

// ----- arena ---------------------------------------------------------------------------------------------------
SX_EXPORT void* sx_arena_create(long long chunk_size) { return new Arena((size_t)chunk_size); }
SX_EXPORT void sx_arena_destroy(void* a) { delete (Arena*)a; }
SX_EXPORT void* sx_arena_alloc(void* a, long long n) { return ((Arena*)a)->alloc((size_t)n, 16); }
SX_EXPORT void* sx_arena_alloc_aligned(void* a, long long n, long long align) { return ((Arena*)a)->alloc((size_t)n, (size_t)align); }
SX_EXPORT void sx_arena_reset(void* a) { ((Arena*)a)->reset(); }
SX_EXPORT long long sx_arena_used(void* a) { return (long long)((Arena*)a)->used(); }
SX_EXPORT long long sx_arena_capacity(void* a) { return (long long)((Arena*)a)->capacity(); }
// out = {used, capacity, chunks, allocations, peak}
SX_EXPORT void sx_arena_stats(void* h, long long* out) {
  auto* a = (Arena*)h;
  out[0] = (long long)a->used(); out[1] = (long long)a->capacity(); out[2] = (long long)a->chunks.size();
  out[3] = (long long)a->n_allocs; out[4] = (long long)a->peak;
}

// ----- slab ----------------------------------------------------------------------------------------------------
SX_EXPORT void* sx_slab_create(long long obj_size, int objs_per_slab) { return new SlabCache((size_t)obj_size, objs_per_slab); }
SX_EXPORT void sx_slab_destroy(void* c) { delete (SlabCache*)c; }
SX_EXPORT void* sx_slab_alloc(void* h) { auto* c = (SlabCache*)h; std::lock_guard<std::mutex> lk(c->mu); return c->alloc_locked(); }
SX_EXPORT int sx_slab_free(void* h, void* p) { auto* c = (SlabCache*)h; std::lock_guard<std::mutex> lk(c->mu); return c->free_locked(p); }
SX_EXPORT int sx_slab_gc(void* c) { return ((SlabCache*)c)->gc(); }
// out = {slabs, free objects, allocations, frees, object size}
SX_EXPORT void sx_slab_stats(void* h, long long* out) {
  auto* c = (SlabCache*)h; std::lock_guard<std::mutex> lk(c->mu);
  out[0] = (long long)c->slabs.size(); out[1] = (long long)c->free_list.size(); out[2] = (long long)c->n_alloc;
  out[3] = (long long)c->n_free; out[4] = (long long)c->obj_size;
}
SX_EXPORT void* sx_slab_local_create(void* cache, int magazine_size) { return new Magazine{(SlabCache*)cache, std::max(magazine_size, 1), {}}; }
SX_EXPORT void* sx_slab_local_alloc(void* h) {
  auto* m = (Magazine*)h;
  if (m->items.empty()) {
    std::lock_guard<std::mutex> lk(m->cache->mu);
    for (int i = 0; i < (m->cap + 1) / 2; ++i) m->items.push_back(m->cache->alloc_locked());
  }
  void* p = m->items.back(); m->items.pop_back(); return p;
}
SX_EXPORT void sx_slab_local_free(void* h, void* p) {
  auto* m = (Magazine*)h;
  m->items.push_back(p);
  if ((int)m->items.size() > m->cap) {
    std::lock_guard<std::mutex> lk(m->cache->mu);
    while ((int)m->items.size() > m->cap / 2) { m->cache->free_locked(m->items.back()); m->items.pop_back(); }
  }
}
SX_EXPORT void sx_slab_local_flush(void* h) {
  auto* m = (Magazine*)h; std::lock_guard<std::mutex> lk(m->cache->mu);
  for (void* p : m->items) m->cache->free_locked(p);
  m->items.clear();
}
SX_EXPORT void sx_slab_local_destroy(void* h) { sx_slab_local_flush(h); delete (Magazine*)h; }

// ----- virtual memory ------------------------------------------------------------------------------------------
SX_EXPORT long long sx_vmem_page_size() { return (long long)sysconf(_SC_PAGESIZE); }
SX_EXPORT void* sx_vmem_reserve(long long n) {
  void* p = mmap(nullptr, (size_t)n, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  return p == MAP_FAILED ? nullptr : p;
}
SX_EXPORT int sx_vmem_commit(void* p, long long n) { return mprotect(p, (size_t)n, PROT_READ | PROT_WRITE); }
SX_EXPORT int sx_vmem_decommit(void* p, long long n) {
  if (madvise(p, (size_t)n, MADV_DONTNEED)) return -1;
  return mprotect(p, (size_t)n, PROT_NONE);
}
SX_EXPORT int sx_vmem_release(void* p, long long n) { return munmap(p, (size_t)n); }
SX_EXPORT int sx_vmem_advise_hugepage(void* p, long long n, int on) { return madvise(p, (size_t)n, on ? MADV_HUGEPAGE : MADV_NOHUGEPAGE); }

// ----- object pool ---------------------------------------------------------------------------------------------
SX_EXPORT void* sx_objpool_create(long long obj_size, int capacity) {
  auto* p = new ObjPool; p->obj_size = (size_t)obj_size; p->capacity = capacity; return p;
}
SX_EXPORT void sx_objpool_clear(void* h) {
  auto* p = (ObjPool*)h; std::lock_guard<std::mutex> lk(p->mu);
  for (void* o : p->all) std::free(o);
  p->all.clear(); p->free_objs.clear();
}
SX_EXPORT void sx_objpool_destroy(void* h) { sx_objpool_clear(h); delete (ObjPool*)h; }
SX_EXPORT int sx_objpool_prealloc(void* h, int n) {
  auto* p = (ObjPool*)h; std::lock_guard<std::mutex> lk(p->mu);
  int made = 0;
  while (made < n && (int)p->all.size() < p->capacity) { void* o = std::calloc(1, p->obj_size); p->all.push_back(o); p->free_objs.push_back(o); ++made; }
  return made;
}
// nullptr when every object of a full pool is out
SX_EXPORT void* sx_objpool_acquire(void* h) {
  auto* p = (ObjPool*)h; std::lock_guard<std::mutex> lk(p->mu);
  if (p->free_objs.empty()) {
    if ((int)p->all.size() >= p->capacity) return nullptr;
    void* o = std::calloc(1, p->obj_size); p->all.push_back(o); return o;
  }
  void* o = p->free_objs.back(); p->free_objs.pop_back(); return o;
}
SX_EXPORT int sx_objpool_release(void* h, void* o) {
  auto* p = (ObjPool*)h; std::lock_guard<std::mutex> lk(p->mu);
  if (std::find(p->all.begin(), p->all.end(), o) == p->all.end()) return -1;
  if (std::find(p->free_objs.begin(), p->free_objs.end(), o) != p->free_objs.end()) return -2;  // double release
  std::memset(o, 0, p->obj_size); p->free_objs.push_back(o); return 0;
}
SX_EXPORT int sx_objpool_available(void* h) {
  auto* p = (ObjPool*)h; std::lock_guard<std::mutex> lk(p->mu);
  return (int)p->free_objs.size() + p->capacity - (int)p->all.size();
}
SX_EXPORT int sx_objpool_capacity(void* h) { return ((ObjPool*)h)->capacity; }

// ----- tiered memory -------------------------------------------------------------------------------------------
SX_EXPORT void* sx_tiered_create(const long long* tier_sizes, int n, const char** names) {
  auto* t = new Tiered;
  for (int i = 0; i < n; ++i) { t->cap.push_back((size_t)tier_sizes[i]); t->used.push_back(0); t->names.push_back(names && names[i] ? names[i] : "tier" + std::to_string(i)); }
  return t;
}
SX_EXPORT void sx_tiered_destroy(void* h) { auto* t = (Tiered*)h; for (auto& b : t->blocks) std::free(b.first); delete t; }
SX_EXPORT void* sx_tiered_alloc(void* h, long long size, int preferred) {
  auto* t = (Tiered*)h; std::lock_guard<std::mutex> lk(t->mu);
  for (int tier = std::max(preferred, 0); tier < (int)t->cap.size(); ++tier)
    if (t->used[tier] + (size_t)size <= t->cap[tier]) {
      void* p = std::aligned_alloc(64, round_up((size_t)size, 64));
      t->used[tier] += (size_t)size; t->blocks[p] = {(size_t)size, tier}; return p;
    }
  return nullptr;
}
SX_EXPORT int sx_tiered_free(void* h, void* p) {
  auto* t = (Tiered*)h; std::lock_guard<std::mutex> lk(t->mu);
  auto it = t->blocks.find(p);
  if (it == t->blocks.end()) return -1;
  t->used[it->second.tier] -= it->second.size; std::free(p); t->blocks.erase(it); return 0;
}
// Accounting moves with the block; the address stays valid. -2 when the target tier has no room.
SX_EXPORT int sx_tiered_migrate(void* h, void* p, int target) {
  auto* t = (Tiered*)h; std::lock_guard<std::mutex> lk(t->mu);
  auto it = t->blocks.find(p);
  if (it == t->blocks.end() || target < 0 || target >= (int)t->cap.size()) return -1;
  if (it->second.tier == target) return 0;
  if (t->used[target] + it->second.size > t->cap[target]) return -2;
  t->used[it->second.tier] -= it->second.size; t->used[target] += it->second.size; it->second.tier = target; return 0;
}
SX_EXPORT int sx_tiered_get_tier(void* h, const void* p) {
  auto* t = (Tiered*)h; std::lock_guard<std::mutex> lk(t->mu);
  auto it = t->blocks.find((void*)p); return it == t->blocks.end() ? -1 : it->second.tier;
}
SX_EXPORT long long sx_tiered_used(void* h, int tier) { auto* t = (Tiered*)h; std::lock_guard<std::mutex> lk(t->mu); return (long long)t->used[tier]; }
SX_EXPORT const char* sx_tiered_name(void* h, int tier) { return ((Tiered*)h)->names[tier].c_str(); }

// ---------------------------------------------------------------------------------------------------------------
// Compression codecs for fp32 buffers. Stream = u32 codec id | u32 block | u64 n | payload.
//   none   raw copy
//   bfp8   per block of `block` values: i8 shared exponent e, then i8 mantissas q with x ~ q * 2^(e - 6)
//   bfp4   same with 4-bit mantissas (two per byte), x ~ q * 2^(e - 2)
//   sparse values with |x| > threshold as (u32 index, f32 value) pairs, the rest decode to zero
// The shared exponent is the smallest e with max|x| < 2^(e + 1), so the largest value uses the full mantissa range.
// ---------------------------------------------------------------------------------------------------------------
namespace {
enum { C_NONE = 0, C_BFP8 = 1, C_BFP4 = 2, C_SPARSE = 3 };
int codec_id(const char* name) {
  std::string s = name ? name : "";
  return s == "none" ? C_NONE : s == "bfp8" ? C_BFP8 : s == "bfp4" ? C_BFP4 : s == "sparse" ? C_SPARSE : -1;
}
int block_exponent(const float* x, size_t n) {
  float m = 0; for (size_t i = 0; i < n; ++i) m = std::max(m, std::fabs(x[i]));
  if (m == 0 || !std::isfinite(m)) return -127;
  int e; std::frexp(m, &e);  // m = f * 2^e, f in [0.5, 1) -> m < 2^e
  return std::max(-127, std::min(127, e - 1));
}
}  // namespace

SX_EXPORT long long sx_compress_bound(const char* codec, long long n, int block) {
  int id = codec_id(codec); if (block <= 0) block = 32;
  long long blocks = (n + block - 1) / block;
  switch (id) {
    case C_NONE: return 16 + 4 * n;
    case C_BFP8: return 16 + blocks + n;
    case C_BFP4: return 16 + blocks + blocks * ((block + 1) / 2);
    case C_SPARSE: return 16 + 8 + 8 * n;
  }
  return -1;
}

SX_EXPORT long long sx_compress(const char* codec, const float* x, long long n, int block, float threshold, void* out, long long cap) {
  int id = codec_id(codec); if (block <= 0) block = 32;
  if (id < 0) return -1;
  if (sx_compress_bound(codec, n, block) > cap) return -2;
  uint8_t* o = (uint8_t*)out; uint32_t hid = (uint32_t)id, hb = (uint32_t)block; uint64_t hn = (uint64_t)n;
  memcpy(o, &hid, 4); memcpy(o + 4, &hb, 4); memcpy(o + 8, &hn, 8);
  size_t k = 16;
  if (id == C_NONE) { memcpy(o + k, x, 4 * (size_t)n); return (long long)(k + 4 * (size_t)n); }
  if (id == C_SPARSE) {
    uint64_t cnt = 0; size_t cnt_at = k; k += 8;
    for (long long i = 0; i < n; ++i) if (std::fabs(x[i]) > threshold) { uint32_t idx = (uint32_t)i; memcpy(o + k, &idx, 4); memcpy(o + k + 4, &x[i], 4); k += 8; ++cnt; }
    memcpy(o + cnt_at, &cnt, 8); return (long long)k;
  }
  const int mant = id == C_BFP8 ? 6 : 2, qmax = id == C_BFP8 ? 127 : 7;
  for (long long b0 = 0; b0 < n; b0 += block) {
    size_t len = (size_t)std::min<long long>(block, n - b0);
    int e = block_exponent(x + b0, len);
    o[k++] = (uint8_t)(int8_t)e;
    float inv = std::ldexp(1.0f, mant - e);
    if (id == C_BFP8) {
      for (size_t i = 0; i < len; ++i) { int q = (int)std::lrint(x[b0 + i] * inv); o[k++] = (uint8_t)(int8_t)std::max(-qmax, std::min(qmax, q)); }
    } else {
      for (size_t i = 0; i < (size_t)block; i += 2) {
        int q0 = i < len ? (int)std::lrint(x[b0 + i] * inv) : 0, q1 = i + 1 < len ? (int)std::lrint(x[b0 + i + 1] * inv) : 0;
        q0 = std::max(-qmax, std::min(qmax, q0)); q1 = std::max(-qmax, std::min(qmax, q1));
        o[k++] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
      }
    }
  }
  return (long long)k;
}

// Returns the element count written, or < 0 on a malformed stream / short output buffer
SX_EXPORT long long sx_decompress(const void* in, long long nbytes, float* y, long long cap) {
  const uint8_t* p = (const uint8_t*)in;
  if (nbytes < 16) return -1;
  uint32_t id, block; uint64_t n; memcpy(&id, p, 4); memcpy(&block, p + 4, 4); memcpy(&n, p + 8, 8);
  if (cap < 0 || n > (uint64_t)cap || block == 0 || block > 65536) return -2;  // header fields come from untrusted bytes
  size_t k = 16;
  if (id == C_NONE) { if (n > ((size_t)nbytes - k) / 4) return -1; memcpy(y, p + k, 4 * n); return (long long)n; }
  if (id == C_SPARSE) {
    uint64_t cnt; if (nbytes < 24) return -1; memcpy(&cnt, p + k, 8); k += 8;
    if (cnt > ((size_t)nbytes - k) / 8) return -1;  // written as a division: 8 * cnt can wrap
    std::fill(y, y + n, 0.0f);
    for (uint64_t i = 0; i < cnt; ++i, k += 8) { uint32_t idx; memcpy(&idx, p + k, 4); if (idx >= n) return -1; memcpy(&y[idx], p + k + 4, 4); }
    return (long long)n;
  }
  if (id != C_BFP8 && id != C_BFP4) return -1;
  const int mant = id == C_BFP8 ? 6 : 2;
  for (uint64_t b0 = 0; b0 < n; b0 += block) {
    size_t len = (size_t)std::min<uint64_t>(block, n - b0);
    if ((size_t)nbytes < k + 1 + (id == C_BFP8 ? len : ((size_t)block + 1) / 2)) return -1;
    int e = (int8_t)p[k++];
    float s = std::ldexp(1.0f, e - mant);
    if (id == C_BFP8) { for (size_t i = 0; i < len; ++i) y[b0 + i] = (float)(int8_t)p[k++] * s; }
    else for (size_t i = 0; i < block; i += 2) {
      uint8_t v = p[k++]; int q0 = (int)(v & 0xF), q1 = (int)(v >> 4);
      if (q0 > 7) q0 -= 16;
      if (q1 > 7) q1 -= 16;
      if (i < len) y[b0 + i] = (float)q0 * s;
      if (i + 1 < len) y[b0 + i + 1] = (float)q1 * s;
    }
  }
  return (long long)n;
}
