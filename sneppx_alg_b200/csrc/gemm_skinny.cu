// G1 for decode-sized inputs (M <= 128 rows of activations against a [N, K] weight): weight streaming on tcgen05 with
// the operands swapped and the reduction split over a thread-block cluster.
//
// The general kernel (gemm_tc.cu) tiles the OUTPUT, so a 64 x 4096 product has 16 tiles and runs on 16 of 148 SMs: the
// weight, which is all of the traffic, streams at a fraction of the HBM rate. Here
//   D^T[n, m] = W[n, :] . X[m, :]     UMMA M = 128 weight rows, UMMA N = M rounded up to 16, fp32 in TMEM
// one CTA owns (128 weight rows, one slice of K); the S CTAs of a cluster own the S slices of the same rows, leave
// their fp32 partial tiles in shared memory and reduce them through distributed shared memory (CTA r sums and writes
// the activation rows m = r, r + S, ...): deterministic, no workspace, no atomics. S is chosen so that tiles x S fills
// the machine in one wave where it can. Two CTAs fit on an SM, each with 3-5 TMA stages in flight.
// The kernel is launched with programmatic stream serialisation: it may become resident while the kernel before it on
// the stream is still running, sets up its barriers and TMEM, and (when the caller says that the weight is not
// produced by earlier kernels: flags bit 0) starts the weight loads of its first stages; everything that depends on
// the predecessor - the activation loads and every store - comes after griddepcontrol.wait.
// (Role in the reference: the batched matmul of its inference engine's decode step, csrc/inference/engine.cpp.)
#include <stdlib.h>
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int SK_BM = 128;       // weight rows per tile
constexpr int SK_BK = 64;        // K elements per stage (one 128-byte swizzle row)
constexpr int SK_THREADS = 192;  // warps 0-3: epilogue (TMEM lane quadrants), warp 4: MMA, warp 5: TMA
constexpr int SK_MAX_STAGES = 6;
constexpr int SK_A_BYTES = SK_BM * SK_BK * 2;

struct SkinnyParams {
  CUtensorMap tmW, tmX;
  void* D;
  const float* bias;
  int* status;
  long long ldd;
  int M, N, K, Mpad, stages, tmem_cols, out_fp32, act, flags;
  float alpha;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Blocks until every kernel this launch depends on has completed and its writes are visible (no-op for a launch
// without a programmatic dependency).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel on the stream start its own prologue (it still waits for this one before reading its results).
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t local_addr, uint32_t rank) {
  uint32_t ra;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(ra)
               : "memory");
  return v;
}

__device__ __forceinline__ float skinny_epilogue(float v, const SkinnyParams& p, int n) {
  v *= p.alpha;
  if (p.bias) v += p.bias[n];
  if (p.act == 1) v = gelu_tanh(v);
  else if (p.act == 2) v = silu(v);
  else if (p.act == 3) v = fmaxf(v, 0.f);
  return v;
}
__device__ __forceinline__ void skinny_store(const SkinnyParams& p, int m, int n, float v) {
  if (p.out_fp32) reinterpret_cast<float*>(p.D)[(long long)m * p.ldd + n] = v;
  else reinterpret_cast<__nv_bfloat16*>(p.D)[(long long)m * p.ldd + n] = __float2bfloat16_rn(v);
}

__global__ void __launch_bounds__(SK_THREADS, 2) gemm_skinny_kernel(const __grid_constant__ SkinnyParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = SK_A_BYTES + p.Mpad * 128;
  uint8_t* sStages = smem;
  float* sP = reinterpret_cast<float*>(smem);   // [Mpad][128] fp32 partial tile, over the stages once they are drained
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + SK_MAX_STAGES;
  uint64_t* tfull = bars + 2 * SK_MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * SK_MAX_STAGES + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int S = (int)cluster_size(), r = (int)cluster_rank();
  const int tile = blockIdx.x / S;
  const int n0 = tile * SK_BM;
  const int kb_total = (p.K + SK_BK - 1) / SK_BK;
  const int per = (kb_total + S - 1) / S;
  const int kb0 = r * per;
  const int kb1 = min(kb_total, kb0 + per);
  const int nk = kb1 > kb0 ? kb1 - kb0 : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < p.stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tfull, 1);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmW);
    tma_prefetch_desc(&p.tmX);
  }
  if (warp == 4) tmem_alloc(tmem_slot, p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 5) {
    if (lane == 0) {
      // weight tiles of the first ring pass may be fetched before the predecessor kernel has finished
      const int pre = (p.flags & 1) ? min(nk, p.stages) : 0;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full[i], stage_bytes);
        tma_load_2d(sStages + i * stage_bytes, &p.tmW, &full[i], (kb0 + i) * SK_BK, n0);
      }
      griddep_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(sStages + i * stage_bytes + SK_A_BYTES, &p.tmX, &full[i], (kb0 + i) * SK_BK, 0);
      for (int i = pre; i < nk; ++i) {
        const int s = i % p.stages;
        if (!mbar_wait(&empty[s], ((i / p.stages) & 1) ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&full[s], stage_bytes);
        uint8_t* st = sStages + s * stage_bytes;
        tma_load_2d(st, &p.tmW, &full[s], (kb0 + i) * SK_BK, n0);
        tma_load_2d(st + SK_A_BYTES, &p.tmX, &full[s], (kb0 + i) * SK_BK, 0);
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && nk > 0) {
      const uint32_t idesc = umma_idesc_f16(SK_BM, p.Mpad, 1, 0, 0);
      bool ok = true;
      for (int i = 0; i < nk; ++i) {
        const int s = i % p.stages;
        if (!mbar_wait(&full[s], (i / p.stages) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a0 = smem_u32(sStages + s * stage_bytes), b0 = a0 + SK_A_BYTES;
#pragma unroll
        for (int k = 0; k < SK_BK / 16; ++k)
          umma_f16_ss(tmem_base, umma_desc_sw128(a0 + k * 32, 16, 1024), umma_desc_sw128(b0 + k * 32, 16, 1024), idesc,
                      (i | k) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(tfull);
    }
  } else {
    // epilogue warps: thread t <-> weight row n0 + t (TMEM lane t)
    const int t = threadIdx.x;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    bool ok = true;
    if (nk > 0) {
      ok = mbar_wait_warp(tfull, 0, s_abort, p.status, ST_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    // fp32 tile -> shared memory as [m][128 n] (the stages are drained: every load was consumed by an MMA that tfull
    // covers); the write-out below then reads whole rows, so that stores to D are 8- or 16-byte pieces of a row
    for (int c = 0; c < p.Mpad / 16; ++c) {
      uint32_t v[16];
      if (ok && nk > 0) {
        tmem_ld16(taddr + c * 16, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) sP[(c * 16 + j) * SK_BM + t] = __uint_as_float(v[j]);
    }
    if (S == 1) asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps only
  }

  // every thread of every CTA of the cluster takes part in both cluster barriers, whatever happened above
  if (S > 1) cluster_sync_all();
  griddep_launch_dependents();
  if (warp < 4) {
    griddep_wait();   // stores (and the bias read) come after the predecessor kernel
    // CTA r owns the activation rows m = r, r + S, ...: sum the S partial tiles (fixed order) and write the row out.
    // Thread layout: 32 float4 column groups x 4 row slots.
    const int q = threadIdx.x & 31, slot = threadIdx.x >> 5;
    const int n = n0 + q * 4;
    const bool vec_ok = n + 3 < p.N && (p.ldd & 3) == 0 && (reinterpret_cast<uintptr_t>(p.D) & 15) == 0;
    for (int m = r + slot * S; m < p.M; m += 4 * S) {
      const uint32_t a = smem_u32(&sP[m * SK_BM + q * 4]);
      float4 v[8];
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s < S) v[s] = S > 1 ? ld_dsmem_f32x4(a, (uint32_t)s) : *reinterpret_cast<const float4*>(&sP[m * SK_BM + q * 4]);
      float4 acc = v[0];
#pragma unroll
      for (int s = 1; s < 8; ++s)
        if (s < S) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
      float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < p.N) o[j] = skinny_epilogue(o[j], p, n + j);
      if (vec_ok) {
        if (p.out_fp32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.D) + (long long)m * p.ldd + n) =
              make_float4(o[0], o[1], o[2], o[3]);
        } else {
          uint2 w;
          w.x = pack_bf16x2(o[0], o[1]);
          w.y = pack_bf16x2(o[2], o[3]);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)m * p.ldd + n) = w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) skinny_store(p, m, n + j, o[j]);
      }
    }
  }
  if (S > 1) cluster_sync_all();

  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

}  // namespace sx
using namespace sx;

// 1 when the product is one this kernel takes: plain [M<=128, K] x [N, K]^T, both K-major, no addend.
extern "C" int sx_gemm_skinny_ok(const SxGemmArgs* a) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("SX_GEMM_SKINNY");   // 0 sends decode-sized products to the general kernel
    enabled = e ? atoi(e) : 1;
  }
  return enabled && a->M >= 1 && a->M <= 128 && a->N >= 128 && a->K >= 256 && a->batch == 1 && !a->a_mn && !a->b_mn &&
         !(a->C && a->beta != 0.f) && !a->tile_group && !a->k_ranges && a->sm_limit == 0 && a->force_bn == 0;
}

// Cluster size (1, 2, 4 or 8): fill the machine in as few waves as possible; cost of a CTA = its K blocks + a fixed
// part. Measured at 64 activation rows on 148 SMs: [6144, 4096] 31.9 / 19.9 / 16.5 / 20.9 us for sizes 1 / 2 / 4 / 8,
// [4096, 4096] 31.3 / 19.3 / 13.5 / 13.1, [28672, 4096] 48.4 / 52.0 / 61.4 / 73.1, [4096, 14336] 89.8 / 49.3 / 29.8 /
// 27.3; the rule below picks the fastest of each. (The occupancy calculator reports one resident CTA per SM for
// cluster launches of this kernel although two fit; the rule counts two.)
extern "C" int sx_gemm_skinny_splits(int N, int K, int sms) {
  static int forced = -1;
  if (forced < 0) {
    const char* e = getenv("SX_SKINNY_SPLITS");   // 1..8 pins the cluster size (measurement aid)
    forced = e ? atoi(e) : 0;
  }
  if (forced >= 1 && forced <= 8) return forced;
  const int tiles = (N + SK_BM - 1) / SK_BM, kb = (K + SK_BK - 1) / SK_BK;
  const int slots = 2 * sms;
  if (tiles >= sms) return 1;   // every SM already has a tile: splitting K would only add reduction work
  int best = 1;
  long long best_cost = -1;
  for (int s = 1; s <= 8; s *= 2) {
    const int per = (kb + s - 1) / s;
    if (s > 1 && per < 4) break;
    const long long cost = (long long)(((long long)tiles * s + slots - 1) / slots) * (per + 6);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

extern "C" int sx_gemm_skinny(const SxGemmArgs* a, cudaStream_t st) {
  if ((a->lda % 8) || (a->ldb % 8) || (a->K % 8) || (reinterpret_cast<uintptr_t>(a->A) & 15) ||
      (reinterpret_cast<uintptr_t>(a->B) & 15))
    return -1;
  SkinnyParams p;
  p.Mpad = (a->M + 15) / 16 * 16;
  {
    uint64_t dims[2] = {(uint64_t)a->K, (uint64_t)a->N};
    uint64_t strides[1] = {(uint64_t)a->ldb * 2};
    uint32_t box[2] = {SK_BK, SK_BM};
    int rc = make_tmap(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->B, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)a->K, (uint64_t)a->M};
    uint64_t strides[1] = {(uint64_t)a->lda * 2};
    uint32_t box[2] = {SK_BK, (uint32_t)p.Mpad};
    int rc = make_tmap(&p.tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->A, dims, strides, box);
    if (rc) return rc;
  }
  const int stage_bytes = SK_A_BYTES + p.Mpad * 128;
  int stages = 98304 / stage_bytes;
  if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
  p.stages = stages;
  p.tmem_cols = p.Mpad <= 32 ? 32 : (p.Mpad <= 64 ? 64 : 128);
  p.D = a->D; p.bias = a->bias; p.status = a->status; p.ldd = a->ldd;
  p.M = a->M; p.N = a->N; p.K = a->K; p.out_fp32 = a->out_fp32; p.act = a->act; p.alpha = a->alpha;
  p.flags = a->flags;
  const int smem = stages * stage_bytes + 1024 + 1024;
  static int smem_set = 0;
  if (smem_set < smem) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 101376) != cudaSuccess)
      return -10;
    smem_set = 101376;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const int S = sx_gemm_skinny_splits(a->N, a->K, sms);
  const int tiles = (a->N + SK_BM - 1) / SK_BM;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * S, 1, 1);
  cfg.blockDim = dim3(SK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static int pdl = -1;
  if (pdl < 0) {
    const char* e = getenv("SX_GEMM_PDL");   // 0: plain stream order (measurement aid)
    pdl = e ? atoi(e) : 1;
  }
  cfg.numAttrs = pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, p) != cudaSuccess) return -11;
  return 0;
}
