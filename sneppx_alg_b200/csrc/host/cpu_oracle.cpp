// Plain C++ CPU oracles for the ops whose GPU kernels need an independent restatement: selective state-space scan,
// router top-k, AdamW. Also the host memory pool / arena / thread pool of the core runtime
// (kernel/memory/allocator.c, mm/arena/arena_alloc.c, kernel/thread/threadpool.c of the reference).
#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <queue>
#include <thread>
#include <vector>

extern "C" {

// y[b,l,h,p] of h_t = exp(dt A) h + dt x B^T ; y = C h + D x.  x [B,L,H,P], dt [B,L,H], A [H], Bm/Cm [B,L,G,N], D [H]
void sx_oracle_ssd(const float* x, const float* dt, const float* A, const float* Bm, const float* Cm, const float* D,
                   float* y, int B, int L, int H, int P, int G, int N) {
  std::vector<float> h((size_t)H * P * N);
  const int rep = H / G;
  for (int b = 0; b < B; ++b) {
    std::fill(h.begin(), h.end(), 0.f);
    for (int l = 0; l < L; ++l)
      for (int hd = 0; hd < H; ++hd) {
        const float d = dt[((size_t)b * L + l) * H + hd];
        const float dA = std::exp(d * A[hd]);
        const float* bv = Bm + (((size_t)b * L + l) * G + hd / rep) * N;
        const float* cv = Cm + (((size_t)b * L + l) * G + hd / rep) * N;
        for (int p = 0; p < P; ++p) {
          const float xv = x[(((size_t)b * L + l) * H + hd) * P + p];
          float* hp = h.data() + ((size_t)hd * P + p) * N;
          float acc = 0.f;
          for (int n = 0; n < N; ++n) {
            hp[n] = hp[n] * dA + d * xv * bv[n];
            acc += hp[n] * cv[n];
          }
          y[(((size_t)b * L + l) * H + hd) * P + p] = acc + (D ? D[hd] * xv : 0.f);
        }
      }
  }
}

// softmax over experts, top-k (lowest index wins ties), renormalised weights
void sx_oracle_router(const float* logits, int T, int E, int k, int* idx, float* w) {
  std::vector<float> p(E);
  for (int t = 0; t < T; ++t) {
    const float* lg = logits + (size_t)t * E;
    const float mx = *std::max_element(lg, lg + E);
    float s = 0;
    for (int e = 0; e < E; ++e) { p[e] = std::exp(lg[e] - mx); s += p[e]; }
    for (int e = 0; e < E; ++e) p[e] /= s;
    float ws = 0;
    for (int r = 0; r < k; ++r) {
      int best = 0;
      for (int e = 1; e < E; ++e)
        if (p[e] > p[best]) best = e;
      idx[(size_t)t * k + r] = best;
      w[(size_t)t * k + r] = p[best];
      ws += p[best];
      p[best] = -1.f;
    }
    for (int r = 0; r < k; ++r) w[(size_t)t * k + r] /= ws;
  }
}

void sx_oracle_adamw(float* p, float* m, float* v, const float* g, long long n, float lr, float b1, float b2, float eps,
                     float wd, int step) {
  const float bc1 = 1.f - std::pow(b1, (float)step), bc2 = 1.f - std::pow(b2, (float)step);
  for (long long i = 0; i < n; ++i) {
    m[i] = b1 * m[i] + (1 - b1) * g[i];
    v[i] = b2 * v[i] + (1 - b2) * g[i] * g[i];
    p[i] -= lr * wd * p[i];
    p[i] -= lr * (m[i] / bc1) / (std::sqrt(v[i] / bc2) + eps);
  }
}

// ---- size-class memory pool with statistics
struct SxPool {
  std::mutex mu;
  std::vector<std::vector<void*>> free_lists = std::vector<std::vector<void*>>(32);
  std::atomic<long long> allocs{0}, hits{0}, bytes_live{0};
};
static int size_class(size_t n) {
  int c = 6;  // 64 B minimum
  while (((size_t)1 << c) < n) ++c;
  return c;
}
void* sx_pool_create() { return new SxPool(); }
void* sx_pool_alloc(void* h, size_t n) {
  SxPool* p = static_cast<SxPool*>(h);
  const int c = size_class(n);
  p->allocs++;
  p->bytes_live += (long long)1 << c;
  {
    std::lock_guard<std::mutex> lk(p->mu);
    if (!p->free_lists[c].empty()) {
      void* r = p->free_lists[c].back();
      p->free_lists[c].pop_back();
      p->hits++;
      return r;
    }
  }
  return aligned_alloc(64, (size_t)1 << c);
}
void sx_pool_free(void* h, void* ptr, size_t n) {
  SxPool* p = static_cast<SxPool*>(h);
  const int c = size_class(n);
  p->bytes_live -= (long long)1 << c;
  std::lock_guard<std::mutex> lk(p->mu);
  p->free_lists[c].push_back(ptr);
}
void sx_pool_stats(void* h, long long* out3) {
  SxPool* p = static_cast<SxPool*>(h);
  out3[0] = p->allocs; out3[1] = p->hits; out3[2] = p->bytes_live;
}
void sx_pool_destroy(void* h) {
  SxPool* p = static_cast<SxPool*>(h);
  for (auto& l : p->free_lists)
    for (void* q : l) free(q);
  delete p;
}
void sx_secure_zero(void* ptr, size_t n) {
  volatile unsigned char* q = static_cast<volatile unsigned char*>(ptr);
  while (n--) *q++ = 0;
}

// ---- thread pool: submit C callbacks, wait for all
struct SxThreadPool {
  std::vector<std::thread> workers;
  std::queue<std::function<void()>> q;
  std::mutex mu;
  std::condition_variable cv, idle;
  int active = 0;
  bool stop = false;
};
void* sx_threadpool_create(int n) {
  SxThreadPool* tp = new SxThreadPool();
  for (int i = 0; i < n; ++i)
    tp->workers.emplace_back([tp] {
      for (;;) {
        std::function<void()> fn;
        {
          std::unique_lock<std::mutex> lk(tp->mu);
          tp->cv.wait(lk, [&] { return tp->stop || !tp->q.empty(); });
          if (tp->q.empty()) return;
          fn = std::move(tp->q.front());
          tp->q.pop();
          tp->active++;
        }
        fn();
        {
          std::lock_guard<std::mutex> lk(tp->mu);
          tp->active--;
        }
        tp->idle.notify_all();
      }
    });
  return tp;
}
typedef void (*sx_task_fn)(void*, long long);
void sx_threadpool_parallel_for(void* h, sx_task_fn fn, void* ctx, long long n) {
  SxThreadPool* tp = static_cast<SxThreadPool*>(h);
  {
    std::lock_guard<std::mutex> lk(tp->mu);
    for (long long i = 0; i < n; ++i) tp->q.push([fn, ctx, i] { fn(ctx, i); });
  }
  tp->cv.notify_all();
  std::unique_lock<std::mutex> lk(tp->mu);
  tp->idle.wait(lk, [&] { return tp->q.empty() && tp->active == 0; });
}
void sx_threadpool_destroy(void* h) {
  SxThreadPool* tp = static_cast<SxThreadPool*>(h);
  {
    std::lock_guard<std::mutex> lk(tp->mu);
    tp->stop = true;
  }
  tp->cv.notify_all();
  for (auto& w : tp->workers) w.join();
  delete tp;
}
}


// ---------------------------------------------------------------------------------------------- conv2d backward
// The same index arithmetic as the CUDA kernels (shared header), run serially: oracle for their tests and the CPU path.
#include "../conv2d_bwd_body.h"

namespace {
struct LoadHost { const float* p; float operator()(long long i) const { return p[i]; } };
}

extern "C" int sx_oracle_conv2d_bwd(const float* x, const float* w, const float* dy, float* dx, float* dw, float* db, int N, int C,
                                    int H, int W, int K, int R, int S, int stride, int pad) {
  if (N < 1 || C < 1 || H < 1 || W < 1 || K < 1 || R < 1 || S < 1 || stride < 1 || pad < 0 || H + 2 * pad < R || W + 2 * pad < S) return -1;
  SxConvDims d{N, C, H, W, K, R, S, (H + 2 * pad - R) / stride + 1, (W + 2 * pad - S) / stride + 1, stride, pad};
  LoadHost ldy{dy}, lw{w}, lx{x};
  if (dx)
    for (int n = 0; n < N; ++n) for (int c = 0; c < C; ++c) for (int h = 0; h < H; ++h) for (int ww = 0; ww < W; ++ww)
      dx[(((long long)n * C + c) * H + h) * W + ww] = sx_conv2d_dx_at(d, ldy, lw, n, c, h, ww);
  if (dw)
    for (int e = 0; e < K * C * R * S; ++e) {
      const int s = e % S, r = (e / S) % R, c = (e / (S * R)) % C, k = e / (S * R * C);
      float acc = 0.f;                     // 256 interleaved partial sums, as the kernel's 256 threads form them
      for (int t = 0; t < 256; ++t) acc += sx_conv2d_dw_partial(d, ldy, lx, k, c, r, s, t, 256);
      dw[e] = acc;
    }
  if (db)
    for (int k = 0; k < K; ++k) {
      float acc = 0.f;
      for (int t = 0; t < 256; ++t) acc += sx_conv2d_db_partial(d, ldy, k, t, 256);
      db[k] = acc;
    }
  return 0;
}


// ---------------------------------------------------------------------------------------------- NPE interpreter
// The instruction semantics of the interpreter kernel (shared header), one thread per row.
#include <vector>
#include "../npe_body.h"

namespace {
struct NpeHostCtx {
  int tid() const { return 0; }
  int nthreads() const { return 1; }
  void sync() const {}
  float sum(float v) const { return v; }
  float max(float v) const { return v; }
};
}

extern "C" int sx_oracle_npe_plan(const int* prog8, int n, long long mem_size, int in_w, int* maxw, int* out_w) {
  if (n < 0 || n > 4096 || in_w < 1) return -1;
  return sx_npe_plan((const SxNpeIns*)prog8, n, mem_size, in_w, maxw, out_w);
}

extern "C" int sx_oracle_npe_run(const int* prog8, int n, const float* mem, long long mem_size, const float* x, long long rows, int in_w,
                                 float* out, int out_w_expected) {
  int maxw = 0, out_w = 0;
  const int rc = sx_oracle_npe_plan(prog8, n, mem_size, in_w, &maxw, &out_w);
  if (rc != 0) return rc;
  if (out_w != out_w_expected || rows < 1) return -2;
  std::vector<float> slots((size_t)(SX_NPE_REGS + 1) * maxw);
  NpeHostCtx ctx;
  for (long long r = 0; r < rows; ++r)
    sx_npe_exec_row((const SxNpeIns*)prog8, n, mem, x + r * in_w, in_w, out + r * out_w, slots.data(), maxw, ctx);
  return 0;
}
