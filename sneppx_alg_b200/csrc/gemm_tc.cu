// G1/G2: persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[b] = act(alpha * A[b] x B[b]^T + bias + beta * C[b])        (fp32 accumulation in TMEM)
//
// A is M x K, B is N x K (both "K-major", i.e. a torch Linear weight is a valid B as is); either
// operand may instead be stored transposed ("MN-major": [K, M] or [K, N] row-major), which covers
// dgrad (dX = dY x W) and wgrad (dW = dY^T x X) without any transposing copy.
// One kernel also serves the grouped (per-expert) GEMMs of the SER MoE layer: a per-M-tile table
// selects which B matrix a row block multiplies (forward / dgrad), and a per-batch reduction range
// restricts K to one expert's token segment (wgrad).
//
// Structure (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (TMEM -> registers -> global). CTA tile 128 x BN x 64, UMMA 128 x BN x 16, smem ring of
// STAGES tiles, two TMEM accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
// Takes the place of the reference's mma.sync / SIMT GEMMs (kernel/cuda/tensor_cuda.cu:28-285) and
// its cuBLAS backward calls (kernel/cuda/autodiff_cuda.cu:28-171).
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmKernelParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  void* D;
  const void* C;
  const float* bias;
  const int* tile_group;  // grouped: per m-block index of the B batch (-1: skip)
  const int* k_ranges;    // per batch [k_begin, k_end)
  int* status;
  long long ldd, ldc, strideD, strideC;
  int M, N, K, batch;
  int a_batched, b_batched;
  int out_fp32, c_fp32, act;
  float alpha, beta;
  int m_blks, n_blks;
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int t, int m_blks, int n_blks, int& b, int& m_blk, int& n_blk) {
  const int per_batch = m_blks * n_blks;
  b = t / per_batch;
  int r = t - b * per_batch;
  constexpr int GM = 8;
  const int group_sz = GM * n_blks;
  const int g = r / group_sz;
  const int first_m = g * GM;
  const int gsz = min(GM, m_blks - first_m);
  const int rr = r - g * group_sz;
  m_blk = first_m + rr % gsz;
  n_blk = rr / gsz;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ GemmKernelParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.batch * p.m_blks * p.n_blks;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, m_blk, n_blk;
        tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        int bsel = b;
        if (p.tile_group) {
          bsel = p.tile_group[m_blk];
          if (bsel < 0) continue;
        }
        int k0 = 0, k1 = p.K;
        if (p.k_ranges) {
          k0 = p.k_ranges[2 * b];
          k1 = p.k_ranges[2 * b + 1];
        }
        const int ab = p.a_batched ? b : 0;
        const int bb = p.b_batched ? bsel : 0;
        const int num_kb = (k1 - k0 + BK - 1) / BK;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int kc = k0 + kb * BK;
          if (A_MN) tma_load_4d(sa, &p.tmA, &full_bar[stage], 0, kc, m_blk * (BM / 64), ab);
          else      tma_load_3d(sa, &p.tmA, &full_bar[stage], kc, m_blk * BM, ab);
          if (B_MN) tma_load_4d(sb, &p.tmB, &full_bar[stage], 0, kc, n_blk * (BN / 64), bb);
          else      tma_load_3d(sb, &p.tmB, &full_bar[stage], kc, n_blk * BN, bb);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        int b, m_blk, n_blk;
        tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        if (p.tile_group && p.tile_group[m_blk] < 0) continue;
        int k0 = 0, k1 = p.K;
        if (p.k_ranges) {
          k0 = p.k_ranges[2 * b];
          k1 = p.k_ranges[2 * b + 1];
        }
        const int num_kb = (k1 - k0 + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (num_kb == 0) {
          // empty reduction range: nothing was accumulated; the epilogue treats it as zeros.
        }
        umma_commit(&tfull_bar[acc]);
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 128 rows)
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      int b, m_blk, n_blk;
      tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
      if (p.tile_group && p.tile_group[m_blk] < 0) continue;
      bool empty_k = false;
      if (p.k_ranges) empty_k = (p.k_ranges[2 * b + 1] <= p.k_ranges[2 * b]);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], acc_phase, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
      const long long crow = (long long)b * p.strideC + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n_blk * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = empty_k ? 0.f : __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || col0 + j < p.N) v[j] += p.bias[col0 + j];
        }
        if (p.beta != 0.f && p.C) {
          if (p.c_fp32) {
            const float* cp = reinterpret_cast<const float*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * cp[j];
          } else {
            const __nv_bfloat16* cp = reinterpret_cast<const __nv_bfloat16*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * __bfloat162float(cp[j]);
          }
        }
        if (p.act == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        } else if (p.act == 2) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
        } else if (p.act == 3) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        if (p.out_fp32) {
          float* dp = reinterpret_cast<float*>(p.D) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = v[j];
          }
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16x2(v[j], v[j + 1]);
              o.y = pack_bf16x2(v[j + 2], v[j + 3]);
              o.z = pack_bf16x2(v[j + 4], v[j + 5]);
              o.w = pack_bf16x2(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(dp + j) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      ++it;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);  // let copies in flight land before freeing
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_cfg(const GemmKernelParams& kp, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_tc_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    attr_set = true;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(kp);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int make_operand_map(CUtensorMap* tm, const void* ptr, int mn, int K, long long ld, int batched, int batch,
                            long long stride, bool mn_major, int tile_mn) {
  if (mn_major) {
    if (mn % 64 != 0) return -20;
    uint64_t dims[4] = {64, (uint64_t)K, (uint64_t)(mn / 64), (uint64_t)(batched ? batch : 1)};
    uint64_t strides[3] = {(uint64_t)ld * 2, 128, (uint64_t)(batched ? stride : (long long)K * ld) * 2};
    uint32_t box[4] = {64, (uint32_t)BK, (uint32_t)(tile_mn / 64), 1};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box);
  } else {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)mn, (uint64_t)(batched ? batch : 1)};
    uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)(batched ? stride : (long long)mn * ld) * 2};
    uint32_t box[3] = {(uint32_t)BK, (uint32_t)tile_mn, 1};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box);
  }
}

}  // namespace sx

extern "C" int sx_gemm_bf16(const SxGemmArgs* a, cudaStream_t st) {
  using namespace sx;
  if (a->M <= 0 || a->N <= 0 || a->batch <= 0) return 0;
  if ((a->lda % 8) || (a->ldb % 8) || (reinterpret_cast<uintptr_t>(a->A) & 15) ||
      (reinterpret_cast<uintptr_t>(a->B) & 15))
    return -1;
  if (a->K % 8) return -2;
  GemmKernelParams kp;
  const int BN = (a->N > 128 || a->force_bn == 256) && a->force_bn != 128 ? 256 : 128;
  const int a_batched = a->strideA != 0 && a->batch > 1;
  const int b_batched = (a->strideB != 0 && a->batch > 1) || a->tile_group != nullptr;
  const int b_nbatch = a->tile_group ? a->num_groups : a->batch;
  // Reduction length seen by the tensor maps: total K rows/cols of the operand storage.
  const int Kfull = a->k_ranges ? a->k_total : a->K;
  int rc = make_operand_map(&kp.tmA, a->A, a->M, Kfull, a->lda, a_batched, a->batch, a->strideA, a->a_mn != 0, BM);
  if (rc) return rc;
  rc = make_operand_map(&kp.tmB, a->B, a->N, Kfull, a->ldb, b_batched, b_nbatch, a->strideB, a->b_mn != 0, BN);
  if (rc) return rc;
  kp.D = a->D;
  kp.C = a->C;
  kp.bias = a->bias;
  kp.tile_group = a->tile_group;
  kp.k_ranges = a->k_ranges;
  kp.status = a->status;
  kp.ldd = a->ldd;
  kp.ldc = a->ldc;
  kp.strideD = a->strideD;
  kp.strideC = a->strideC;
  kp.M = a->M;
  kp.N = a->N;
  kp.K = a->K;
  kp.batch = a->batch;
  kp.a_batched = a_batched;
  kp.b_batched = b_batched;
  kp.out_fp32 = a->out_fp32;
  kp.c_fp32 = a->c_fp32;
  kp.act = a->act;
  kp.alpha = a->alpha;
  kp.beta = a->beta;
  kp.m_blks = (a->M + BM - 1) / BM;
  kp.n_blks = (a->N + BN - 1) / BN;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  static int cached_sms[16] = {0};
  if (dev < 16 && cached_sms[dev] == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cached_sms[dev] = sms;
  }
  if (dev < 16) sms = cached_sms[dev];
  if (a->sm_limit > 0 && a->sm_limit < sms) sms = a->sm_limit;
  const long long tiles = (long long)kp.batch * kp.m_blks * kp.n_blks;
  const int grid = (int)(tiles < sms ? tiles : sms);
  const int am = a->a_mn != 0, bm = a->b_mn != 0;
  if (BN == 256) {
    if (!am && !bm) return launch_cfg<256, false, false>(kp, grid, st);
    if (!am && bm) return launch_cfg<256, false, true>(kp, grid, st);
    if (am && !bm) return launch_cfg<256, true, false>(kp, grid, st);
    return launch_cfg<256, true, true>(kp, grid, st);
  } else {
    if (!am && !bm) return launch_cfg<128, false, false>(kp, grid, st);
    if (!am && bm) return launch_cfg<128, false, true>(kp, grid, st);
    if (am && !bm) return launch_cfg<128, true, false>(kp, grid, st);
    return launch_cfg<128, true, true>(kp, grid, st);
  }
}
