// Memory security layer (S1) and in-process tamper monitors (S3), host side.
//
//   leak detector      every tracked allocation carries (size, file, line, function, sequence number); a check lists
//                      what is still live above a size threshold, with totals / peak / counts
//   quarantine         freed blocks are poisoned (0xDD) and parked in a FIFO until a byte budget is exceeded; a
//                      block that was written while parked (use after free) is reported when it leaves
//   pointer signing    64-bit keyed tag of (pointer, key slot) - SipHash-2-4 over the address with a per-process key -
//                      for indirect-call tables; verify is constant time
//   control-flow set   allowed indirect-call targets; validate() says whether a pointer is one of them
//   shadow stack       return addresses pushed on call and compared on return
//   canary pool        random 64-bit canaries handed out per thread / frame and checked later
//   guard-page pool    page-aligned allocations with an inaccessible page before and after (mmap + mprotect); the
//                      user range ends flush against the trailing guard page
//   memory pressure    byte budget with soft / hard limits
//   metadata masking   XOR stream keyed per process for allocator headers kept in memory
//   code-tamper        FNV-1a/64 digests of registered memory regions, re-checked on demand
//   heap sentinels     64-bit words placed behind allocations and scanned in bulk
//   W^X                flips a page range between read-write and read-execute, never both
// Behavioural counterparts: security/memory/memory_leak_detector.c, memory_hardening.c (quarantine, heap metadata
// encryption, W^X, PAC, CFG, shadow stack, TLS canaries, guard pool, memory pressure) and
// security/monitor/monitor_advanced.c (code tamper detector, heap corruption sentinels, return-address check).
#include <sys/mman.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <random>
#include <set>
#include <string>
#include <vector>

namespace {

uint64_t rotl(uint64_t x, int b) { return (x << b) | (x >> (64 - b)); }

uint64_t siphash24(const uint8_t k[16], const uint8_t* in, size_t n) {
  uint64_t k0, k1;
  std::memcpy(&k0, k, 8);
  std::memcpy(&k1, k + 8, 8);
  uint64_t v0 = 0x736f6d6570736575ull ^ k0, v1 = 0x646f72616e646f6dull ^ k1, v2 = 0x6c7967656e657261ull ^ k0,
           v3 = 0x7465646279746573ull ^ k1;
  auto round = [&] {
    v0 += v1; v1 = rotl(v1, 13); v1 ^= v0; v0 = rotl(v0, 32);
    v2 += v3; v3 = rotl(v3, 16); v3 ^= v2;
    v0 += v3; v3 = rotl(v3, 21); v3 ^= v0;
    v2 += v1; v1 = rotl(v1, 17); v1 ^= v2; v2 = rotl(v2, 32);
  };
  const size_t end = n - n % 8;
  for (size_t i = 0; i < end; i += 8) {
    uint64_t m;
    std::memcpy(&m, in + i, 8);
    v3 ^= m;
    round();
    round();
    v0 ^= m;
  }
  uint64_t b = (uint64_t)n << 56;
  for (size_t i = 0; i < n % 8; ++i) b |= (uint64_t)in[end + i] << (8 * i);
  v3 ^= b;
  round();
  round();
  v0 ^= b;
  v2 ^= 0xff;
  for (int i = 0; i < 4; ++i) round();
  return v0 ^ v1 ^ v2 ^ v3;
}

uint64_t random64() {
  static std::mutex mu;
  static std::mt19937_64 gen{[] {
    std::random_device rd;
    return ((uint64_t)rd() << 32) ^ rd() ^ (uint64_t)getpid();
  }()};
  std::lock_guard<std::mutex> lk(mu);
  return gen();
}

uint64_t fnv1a(const uint8_t* p, size_t n) {
  uint64_t h = 1469598103934665603ull;
  for (size_t i = 0; i < n; ++i) {
    h ^= p[i];
    h *= 1099511628211ull;
  }
  return h;
}

// ---------------------------------------------------------------- leak detector
struct LeakEntry {
  size_t size;
  std::string file, func;
  int line;
  uint64_t seq;
};
struct LeakState {
  std::mutex mu;
  std::map<uintptr_t, LeakEntry> live;
  bool enabled = true;
  size_t threshold = 0;
  uint64_t seq = 0, allocs = 0, frees = 0, unknown_frees = 0;
  size_t live_bytes = 0, peak_bytes = 0, total_bytes = 0;
} g_leak;

// ---------------------------------------------------------------- quarantine
struct Quarantine {
  struct Item {
    uint8_t* p;
    size_t n;
  };
  std::mutex mu;
  std::deque<Item> fifo;
  size_t bytes = 0, budget;
  uint64_t uaf_detected = 0, released = 0;
};

struct GuardAlloc {
  uint8_t* base;
  size_t total, user;
};
struct GuardPool {
  std::mutex mu;
  std::map<uintptr_t, GuardAlloc> live;
  size_t page;
};

struct TamperRegion {
  const uint8_t* p;
  size_t n;
  uint64_t digest;
  bool active;
};
std::mutex g_tamper_mu;
std::vector<TamperRegion> g_tamper;

}  // namespace

extern "C" {

// ================================================================= leak detector
void sx_leak_reset(void) {
  std::lock_guard<std::mutex> lk(g_leak.mu);
  g_leak.live.clear();
  g_leak.seq = g_leak.allocs = g_leak.frees = g_leak.unknown_frees = 0;
  g_leak.live_bytes = g_leak.peak_bytes = g_leak.total_bytes = 0;
}
void sx_leak_enable(int on) { g_leak.enabled = on != 0; }
void sx_leak_set_threshold(long long bytes) { g_leak.threshold = bytes > 0 ? (size_t)bytes : 0; }
int sx_leak_track_alloc(void* p, size_t n, const char* file, int line, const char* func) {
  if (!p || !g_leak.enabled) return -1;
  std::lock_guard<std::mutex> lk(g_leak.mu);
  g_leak.live[(uintptr_t)p] = LeakEntry{n, file ? file : "", func ? func : "", line, ++g_leak.seq};
  g_leak.allocs++;
  g_leak.live_bytes += n;
  g_leak.total_bytes += n;
  g_leak.peak_bytes = std::max(g_leak.peak_bytes, g_leak.live_bytes);
  return 0;
}
// 0 tracked and removed, 1 pointer was never tracked (double free or foreign pointer)
int sx_leak_track_free(void* p) {
  if (!p || !g_leak.enabled) return -1;
  std::lock_guard<std::mutex> lk(g_leak.mu);
  auto it = g_leak.live.find((uintptr_t)p);
  if (it == g_leak.live.end()) {
    g_leak.unknown_frees++;
    return 1;
  }
  g_leak.live_bytes -= it->second.size;
  g_leak.frees++;
  g_leak.live.erase(it);
  return 0;
}
void* sx_leak_malloc(size_t n, const char* file, int line, const char* func) {
  void* p = std::malloc(n);
  if (p) sx_leak_track_alloc(p, n, file, line, func);
  return p;
}
void sx_leak_free(void* p) {
  if (!p) return;
  sx_leak_track_free(p);
  std::free(p);
}
void* sx_leak_realloc(void* p, size_t n, const char* file, int line, const char* func) {
  if (p) sx_leak_track_free(p);
  void* q = std::realloc(p, n);
  if (q) sx_leak_track_alloc(q, n, file, line, func);
  return q;
}
// out7: live blocks, live bytes, peak bytes, total bytes, allocations, frees, frees of unknown pointers
void sx_leak_stats(long long* out7) {
  std::lock_guard<std::mutex> lk(g_leak.mu);
  out7[0] = (long long)g_leak.live.size();
  out7[1] = (long long)g_leak.live_bytes;
  out7[2] = (long long)g_leak.peak_bytes;
  out7[3] = (long long)g_leak.total_bytes;
  out7[4] = (long long)g_leak.allocs;
  out7[5] = (long long)g_leak.frees;
  out7[6] = (long long)g_leak.unknown_frees;
}
// Writes one line per live block at or above the threshold ("seq size file:line func\n", oldest first) into buf;
// returns the number of such blocks (which may exceed what fitted).
int sx_leak_check(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lk(g_leak.mu);
  std::vector<const LeakEntry*> v;
  for (auto& kv : g_leak.live)
    if (kv.second.size >= g_leak.threshold) v.push_back(&kv.second);
  std::sort(v.begin(), v.end(), [](const LeakEntry* a, const LeakEntry* b) { return a->seq < b->seq; });
  size_t off = 0;
  if (buf && cap) buf[0] = 0;
  for (auto* e : v) {
    char line[512];
    const int n = std::snprintf(line, sizeof line, "%llu %zu %s:%d %s\n", (unsigned long long)e->seq, e->size, e->file.c_str(),
                                e->line, e->func.c_str());
    if (buf && n > 0 && off + (size_t)n + 1 <= cap) {
      std::memcpy(buf + off, line, (size_t)n + 1);
      off += (size_t)n;
    }
  }
  return (int)v.size();
}

// ================================================================= quarantine
void* sx_quarantine_create(size_t budget_bytes) {
  Quarantine* q = new Quarantine();
  q->budget = budget_bytes;
  return q;
}
static int quarantine_release_one(Quarantine* q) {
  auto it = q->fifo.front();
  q->fifo.pop_front();
  q->bytes -= it.n;
  int dirty = 0;
  for (size_t i = 0; i < it.n; ++i)
    if (it.p[i] != 0xDD) {
      dirty = 1;
      break;
    }
  if (dirty) q->uaf_detected++;
  q->released++;
  std::free(it.p);
  return dirty;
}
// Takes ownership of a malloc'd block instead of freeing it. Returns how many parked blocks that were found written
// to (use after free) left the quarantine because of this call.
int sx_quarantine_add(void* h, void* p, size_t n) {
  Quarantine* q = static_cast<Quarantine*>(h);
  if (!p) return 0;
  std::memset(p, 0xDD, n);
  std::lock_guard<std::mutex> lk(q->mu);
  q->fifo.push_back({static_cast<uint8_t*>(p), n});
  q->bytes += n;
  int dirty = 0;
  while (q->bytes > q->budget && !q->fifo.empty()) dirty += quarantine_release_one(q);
  return dirty;
}
// 1 when p lies inside a parked block (a dangling pointer), else 0
int sx_quarantine_contains(void* h, const void* p) {
  Quarantine* q = static_cast<Quarantine*>(h);
  std::lock_guard<std::mutex> lk(q->mu);
  for (auto& it : q->fifo)
    if ((const uint8_t*)p >= it.p && (const uint8_t*)p < it.p + it.n) return 1;
  return 0;
}
// out4: parked blocks, parked bytes, blocks released, use-after-free detections
void sx_quarantine_stats(void* h, long long* out4) {
  Quarantine* q = static_cast<Quarantine*>(h);
  std::lock_guard<std::mutex> lk(q->mu);
  out4[0] = (long long)q->fifo.size();
  out4[1] = (long long)q->bytes;
  out4[2] = (long long)q->released;
  out4[3] = (long long)q->uaf_detected;
}
int sx_quarantine_drain(void* h) {
  Quarantine* q = static_cast<Quarantine*>(h);
  std::lock_guard<std::mutex> lk(q->mu);
  int dirty = 0;
  while (!q->fifo.empty()) dirty += quarantine_release_one(q);
  return dirty;
}
void sx_quarantine_destroy(void* h) {
  sx_quarantine_drain(h);
  delete static_cast<Quarantine*>(h);
}

// ================================================================= pointer signing / CFG / shadow stack / canaries
struct SxPac {
  uint8_t keys[4][16];
};
void* sx_pac_create(void) {
  SxPac* p = new SxPac();
  for (auto& k : p->keys)
    for (int i = 0; i < 16; i += 8) {
      const uint64_t r = random64();
      std::memcpy(k + i, &r, 8);
    }
  return p;
}
void sx_pac_destroy(void* h) { delete static_cast<SxPac*>(h); }
unsigned long long sx_pac_sign(void* h, const void* ptr, int key_idx) {
  const uintptr_t a = (uintptr_t)ptr;
  return siphash24(static_cast<SxPac*>(h)->keys[key_idx & 3], reinterpret_cast<const uint8_t*>(&a), sizeof a);
}
int sx_pac_verify(void* h, const void* ptr, unsigned long long sig, int key_idx) {
  const unsigned long long want = sx_pac_sign(h, ptr, key_idx);
  unsigned long long d = want ^ sig;       // constant time: no early exit on the first differing byte
  d |= d >> 32; d |= d >> 16; d |= d >> 8;
  return (d & 0xff) == 0 ? 1 : 0;
}

struct SxCfg {
  std::mutex mu;
  std::set<uintptr_t> targets;
  uint64_t violations = 0;
};
void* sx_cfg_create(void) { return new SxCfg(); }
void sx_cfg_destroy(void* h) { delete static_cast<SxCfg*>(h); }
int sx_cfg_add_target(void* h, const void* t) {
  SxCfg* c = static_cast<SxCfg*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  return c->targets.insert((uintptr_t)t).second ? 0 : 1;
}
int sx_cfg_validate(void* h, const void* t) {
  SxCfg* c = static_cast<SxCfg*>(h);
  std::lock_guard<std::mutex> lk(c->mu);
  if (c->targets.count((uintptr_t)t)) return 1;
  c->violations++;
  return 0;
}
long long sx_cfg_violations(void* h) { return (long long)static_cast<SxCfg*>(h)->violations; }

struct SxShadow {
  std::vector<uintptr_t> st;
  size_t cap;
  uint64_t mismatches = 0;
};
void* sx_shadow_create(size_t cap) {
  SxShadow* s = new SxShadow();
  s->cap = cap ? cap : 4096;
  return s;
}
void sx_shadow_destroy(void* h) { delete static_cast<SxShadow*>(h); }
int sx_shadow_push(void* h, unsigned long long ret) {
  SxShadow* s = static_cast<SxShadow*>(h);
  if (s->st.size() >= s->cap) return -1;
  s->st.push_back((uintptr_t)ret);
  return 0;
}
// 1 match, 0 mismatch (return address was changed), -1 empty
int sx_shadow_pop_check(void* h, unsigned long long ret) {
  SxShadow* s = static_cast<SxShadow*>(h);
  if (s->st.empty()) return -1;
  const uintptr_t want = s->st.back();
  s->st.pop_back();
  if (want == (uintptr_t)ret) return 1;
  s->mismatches++;
  return 0;
}
long long sx_shadow_depth(void* h) { return (long long)static_cast<SxShadow*>(h)->st.size(); }

struct SxCanaryPool {
  std::mutex mu;
  std::set<uint64_t> live;
};
void* sx_canary_pool_create(void) { return new SxCanaryPool(); }
void sx_canary_pool_destroy(void* h) { delete static_cast<SxCanaryPool*>(h); }
unsigned long long sx_canary_alloc(void* h) {
  SxCanaryPool* p = static_cast<SxCanaryPool*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  uint64_t c;
  do {
    c = random64() & ~0xffull;       // low byte zero: a string overflow cannot copy the canary through
  } while (c == 0 || !p->live.insert(c).second);
  return c;
}
// 1 when the value is a live canary of this pool (and retires it), else 0
int sx_canary_check(void* h, unsigned long long c) {
  SxCanaryPool* p = static_cast<SxCanaryPool*>(h);
  std::lock_guard<std::mutex> lk(p->mu);
  return p->live.erase(c) ? 1 : 0;
}

// ================================================================= guard-page pool
void* sx_guard_pool_create(void) {
  GuardPool* g = new GuardPool();
  g->page = (size_t)sysconf(_SC_PAGESIZE);
  return g;
}
void* sx_guard_pool_alloc(void* h, size_t n) {
  GuardPool* g = static_cast<GuardPool*>(h);
  if (n == 0) return nullptr;
  const size_t body = (n + g->page - 1) / g->page * g->page;
  const size_t total = body + 2 * g->page;
  uint8_t* base = static_cast<uint8_t*>(mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0));
  if (base == MAP_FAILED) return nullptr;
  if (mprotect(base, g->page, PROT_NONE) != 0 || mprotect(base + g->page + body, g->page, PROT_NONE) != 0) {
    munmap(base, total);
    return nullptr;
  }
  uint8_t* user = base + g->page + body - n;      // the last byte touches the trailing guard page
  user = reinterpret_cast<uint8_t*>((uintptr_t)user & ~(uintptr_t)15);
  std::lock_guard<std::mutex> lk(g->mu);
  g->live[(uintptr_t)user] = GuardAlloc{base, total, n};
  return user;
}
int sx_guard_pool_free(void* h, void* p) {
  GuardPool* g = static_cast<GuardPool*>(h);
  std::lock_guard<std::mutex> lk(g->mu);
  auto it = g->live.find((uintptr_t)p);
  if (it == g->live.end()) return -1;
  munmap(it->second.base, it->second.total);
  g->live.erase(it);
  return 0;
}
// Distance in bytes from p to the first inaccessible byte after it (-1: not a pool pointer)
long long sx_guard_pool_room(void* h, void* p) {
  GuardPool* g = static_cast<GuardPool*>(h);
  std::lock_guard<std::mutex> lk(g->mu);
  auto it = g->live.find((uintptr_t)p);
  if (it == g->live.end()) return -1;
  return (long long)((it->second.base + it->second.total - g->page) - static_cast<uint8_t*>(p));
}
long long sx_guard_pool_live(void* h) { return (long long)static_cast<GuardPool*>(h)->live.size(); }
void sx_guard_pool_destroy(void* h) {
  GuardPool* g = static_cast<GuardPool*>(h);
  for (auto& kv : g->live) munmap(kv.second.base, kv.second.total);
  delete g;
}

// ================================================================= W^X, memory pressure, metadata masking
// mode 0: read-write, 1: read-execute. The range must be page aligned. A page is never writable and executable.
int sx_mem_set_mode(void* addr, size_t n, int mode) {
  const size_t page = (size_t)sysconf(_SC_PAGESIZE);
  if (((uintptr_t)addr % page) || n == 0) return -1;
  return mprotect(addr, (n + page - 1) / page * page, mode == 1 ? (PROT_READ | PROT_EXEC) : (PROT_READ | PROT_WRITE));
}
void* sx_mem_alloc_pages(size_t n) {
  void* p = mmap(nullptr, n, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
  return p == MAP_FAILED ? nullptr : p;
}
int sx_mem_free_pages(void* p, size_t n) { return munmap(p, n); }

struct SxPressure {
  std::atomic<long long> used{0};
  long long soft, hard;
  std::atomic<long long> rejected{0};
};
void* sx_pressure_create(long long soft, long long hard) {
  SxPressure* p = new SxPressure();
  p->soft = soft;
  p->hard = hard;
  return p;
}
void sx_pressure_destroy(void* h) { delete static_cast<SxPressure*>(h); }
// 0 accepted, 1 accepted above the soft limit (caller should shed load), -1 rejected (would pass the hard limit)
int sx_pressure_reserve(void* h, long long n) {
  SxPressure* p = static_cast<SxPressure*>(h);
  const long long now = p->used.fetch_add(n) + n;
  if (now > p->hard) {
    p->used.fetch_sub(n);
    p->rejected.fetch_add(1);
    return -1;
  }
  return now > p->soft ? 1 : 0;
}
void sx_pressure_release(void* h, long long n) { static_cast<SxPressure*>(h)->used.fetch_sub(n); }
long long sx_pressure_used(void* h) { return static_cast<SxPressure*>(h)->used.load(); }
long long sx_pressure_rejected(void* h) { return static_cast<SxPressure*>(h)->rejected.load(); }

// XOR stream derived from a 16-byte key and the block's address: the same call masks and unmasks.
void sx_metadata_mask(const unsigned char* key16, void* data, size_t n, unsigned long long tweak) {
  uint8_t* d = static_cast<uint8_t*>(data);
  for (size_t i = 0; i < n; i += 8) {
    const uint64_t ctr[2] = {tweak, (uint64_t)i};
    const uint64_t ks = siphash24(key16, reinterpret_cast<const uint8_t*>(ctr), sizeof ctr);
    for (size_t j = 0; j < 8 && i + j < n; ++j) d[i + j] ^= (uint8_t)(ks >> (8 * j));
  }
}

// ================================================================= code-tamper regions and heap sentinels
int sx_tamper_add_region(const void* p, size_t n) {
  std::lock_guard<std::mutex> lk(g_tamper_mu);
  g_tamper.push_back({static_cast<const uint8_t*>(p), n, fnv1a(static_cast<const uint8_t*>(p), n), true});
  return (int)g_tamper.size() - 1;
}
int sx_tamper_remove_region(int i) {
  std::lock_guard<std::mutex> lk(g_tamper_mu);
  if (i < 0 || (size_t)i >= g_tamper.size() || !g_tamper[(size_t)i].active) return -1;
  g_tamper[(size_t)i].active = false;
  return 0;
}
// 1 unchanged, 0 modified since registration, -1 unknown region
int sx_tamper_check(int i) {
  std::lock_guard<std::mutex> lk(g_tamper_mu);
  if (i < 0 || (size_t)i >= g_tamper.size() || !g_tamper[(size_t)i].active) return -1;
  return fnv1a(g_tamper[(size_t)i].p, g_tamper[(size_t)i].n) == g_tamper[(size_t)i].digest ? 1 : 0;
}
// number of registered regions whose contents changed
int sx_tamper_check_all(void) {
  std::lock_guard<std::mutex> lk(g_tamper_mu);
  int bad = 0;
  for (auto& r : g_tamper)
    if (r.active && fnv1a(r.p, r.n) != r.digest) ++bad;
  return bad;
}
void sx_tamper_reset(void) {
  std::lock_guard<std::mutex> lk(g_tamper_mu);
  g_tamper.clear();
}

static std::atomic<uint64_t> g_sentinel{0xDEADC0DEFEEDFACEull};
void sx_sentinel_set_value(unsigned long long v) { g_sentinel.store(v); }
// The allocation must have 8 spare bytes behind its `n` user bytes.
void sx_sentinel_apply(void* alloc, size_t n) {
  const uint64_t v = g_sentinel.load();
  std::memcpy(static_cast<uint8_t*>(alloc) + n, &v, 8);
}
int sx_sentinel_check(const void* alloc, size_t n) {
  uint64_t v;
  std::memcpy(&v, static_cast<const uint8_t*>(alloc) + n, 8);
  return v == g_sentinel.load() ? 1 : 0;
}
// how many of the `count` allocations have a damaged sentinel
int sx_sentinel_scan(void* const* allocs, const size_t* sizes, int count) {
  int bad = 0;
  for (int i = 0; i < count; ++i)
    if (!sx_sentinel_check(allocs[i], sizes[i])) ++bad;
  return bad;
}
int sx_ret_addr_verify(const void* got, const void* expected) { return got == expected ? 1 : 0; }

}  // extern "C"
