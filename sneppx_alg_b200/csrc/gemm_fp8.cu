// Q2 (fp8 x fp8): block-scaled e4m3 GEMM on tcgen05 `kind::f8f6f4`.
//
//   Y[M, N] = (Xq * sx)[M, K] x (Wq * sw)[N, K]^T        Xq, Wq: e4m3; sx: fp32 [M, K/128] (1 x 128 blocks);
//                                                        sw: fp32 [ceil(N/128), K/128] (128 x 128 blocks)
//
// The weights are the MMA's A operand ("swap AB"): a CTA owns 128 weight rows (TMEM lanes) and a tile of BT tokens
// (TMEM columns), so a decode step with a few dozen tokens still fills the 128-row MMA and reads every weight byte
// exactly once. Because the scale product changes every 128 elements of K, each 128-wide k-block is accumulated on
// its own in one of two TMEM buffers (4 MMAs of K = 32) and promoted by the four epilogue warps into fp32 registers
// with its scale (acc += sw[nb, kb] * sx[token, kb] * partial) while the next k-block runs in the other buffer.
// Operand tiles are exactly one 128-byte swizzle row wide (128 fp8 = 128 B), loaded by TMA. With split-K several CTAs
// share a tile's reduction and add fp32 partials into a zeroed workspace that a second kernel converts.
// Grouped form (SER experts, G2 in fp8): the token rows are expert-sorted with every expert's segment padded to
// 128 rows; `tile_group[t]` names the expert of token tile t (-1: unused tile, its output rows are zero-filled).
// The experts' weights are one stacked [E * N, K] tensor (N a multiple of 128, so a 128-row weight tile never
// straddles two experts) with scales [E * N/128, K/128]; a CTA simply offsets its weight-row and scale-row
// coordinates by the tile's expert.
// The reference has e4m3 quantise / dequantise kernels only (kernel/quantization/quantize_cuda.cu,
// kernel/quantization/quantize_fp8.c); block-scaled fp8 experts are what its DeepSeek-shape preset implies.
#include "tc_common.cuh"
#include "common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int F8_BK = 128;        // bytes == elements per k-block
constexpr int F8_THREADS = 192;   // warp 0 TMA, warp 1 MMA, warps 2..5 promotion + epilogue

struct F8Params {
  CUtensorMap tmW, tmX;
  const float* sw;       // [n_blks, kblks]
  const float* sx;       // [M, kblks]
  const float* bias;     // optional [N]
  __nv_bfloat16* D;      // [M, N] (splits == 1)
  float* work;           // [M, N] fp32, zeroed (splits > 1)
  long long ldd;
  int M, N, K, kblks, splits;
  int* status;
  const int* tile_group;   // grouped form: expert of each 128-token tile (BT == 128), else nullptr
};

template <int BT>
struct F8Cfg {
  static constexpr int W_BYTES = 128 * F8_BK;
  static constexpr int X_BYTES = BT * F8_BK;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int SCALE_FLOATS = 16384;             // activation scales of the CTA's (k range, token tile), 64 KB
  static constexpr int STAGES = (150 * 1024) / STAGE_BYTES > 8 ? 8 : (150 * 1024) / STAGE_BYTES;
  static constexpr int OFF_SCALE = STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_SCALE + SCALE_FLOATS * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
};

template <int BT>
__global__ void __launch_bounds__(F8_THREADS, 1) gemm_f8_kernel(const __grid_constant__ F8Params p) {
  using Cfg = F8Cfg<BT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  float* s_sx = reinterpret_cast<float*>(smem + Cfg::OFF_SCALE);   // [k-block of this CTA][token of the tile]
  uint64_t* full_bar = bars;                    // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;     // [STAGES]
  uint64_t* tfull = bars + 2 * Cfg::STAGES;     // [2]
  uint64_t* tempty = tfull + 2;                 // [2], 4 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TCOLS = 2 * BT < 32 ? 32 : 2 * BT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmW);
    tma_prefetch_desc(&p.tmX);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TCOLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int nb = blockIdx.x, tb = blockIdx.y, sp = blockIdx.z;
  const int per = (p.kblks + p.splits - 1) / p.splits;
  const int kb0 = sp * per, kb1 = min(p.kblks, kb0 + per);
  const int grp = p.tile_group ? p.tile_group[tb] : 0;
  const int nkb = grp < 0 ? 0 : max(kb1 - kb0, 0);          // unused tile: no loads, no MMAs, zero output
  const int w_row0 = grp * (p.tile_group ? p.N : 0) + nb * 128;     // row of the stacked weight tensor
  const int s_row = grp * (p.tile_group ? (p.N + 127) / 128 : 0) + nb;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        uint8_t* sw_ = smem + stage * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
        tma_load_2d(sw_, &p.tmW, &full_bar[stage], (kb0 + i) * F8_BK, w_row0);
        tma_load_2d(sw_ + Cfg::W_BYTES, &p.tmX, &full_bar[stage], (kb0 + i) * F8_BK, tb * BT);
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f8(128, BT, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i) {
        const int buf = i & 1;
        if (!mbar_wait(&tempty[buf], ((i >> 1) & 1) ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        if (!mbar_wait(&full_bar[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES), sb = sa + Cfg::W_BYTES;
#pragma unroll
        for (int k = 0; k < F8_BK / 32; ++k)
          umma_f8_ss(tmem_base + buf * BT, umma_desc_sw128(sa + k * 32, 16, 1024), umma_desc_sw128(sb + k * 32, 16, 1024),
                     idesc, k ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        umma_commit(&tfull[buf]);
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ promotion + epilogue: lane = weight row
    const int q = warp & 3;
    const int n = nb * 128 + q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float acc[BT];
#pragma unroll
    for (int j = 0; j < BT; ++j) acc[j] = 0.f;
    bool ok = true;
    const int tok0 = tb * BT;
    // Stage the activation scales of this CTA's k range, transposed to [k-block][token], so that a k-block's BT
    // scales are one contiguous run read with 16-byte shared loads (identical for every lane: broadcast).
    const bool staged = nkb * BT <= Cfg::SCALE_FLOATS;
    if (staged) {
      const int t4 = threadIdx.x - 64;   // 0..127 over the four promotion warps
      for (int e = t4; e < nkb * BT; e += 128) {
        const int j = e % BT, i = e / BT;     // consecutive threads write consecutive shared-memory words
        const int tok = tok0 + j;
        s_sx[i * BT + j] = tok < p.M ? p.sx[(long long)tok * p.kblks + kb0 + i] : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four promotion warps only; no wait can abort before this point
    }
    for (int i = 0; i < nkb && ok; ++i) {
      const int buf = i & 1, kb = kb0 + i;
      const float swv = p.sw[(long long)s_row * p.kblks + kb];
      if (!mbar_wait_warp(&tfull[buf], (i >> 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + buf * BT + c * 32 + lane_addr, v);
        tmem_ld_wait();
        if (staged) {
          const float4* sp4 = reinterpret_cast<const float4*>(s_sx + i * BT + c * 32);
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 s4 = sp4[j >> 2];
            acc[c * 32 + j] = fmaf(__uint_as_float(v[j]), swv * s4.x, acc[c * 32 + j]);
            acc[c * 32 + j + 1] = fmaf(__uint_as_float(v[j + 1]), swv * s4.y, acc[c * 32 + j + 1]);
            acc[c * 32 + j + 2] = fmaf(__uint_as_float(v[j + 2]), swv * s4.z, acc[c * 32 + j + 2]);
            acc[c * 32 + j + 3] = fmaf(__uint_as_float(v[j + 3]), swv * s4.w, acc[c * 32 + j + 3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = tok0 + c * 32 + j;
            const float sxv = tok < p.M ? __ldg(p.sx + (long long)tok * p.kblks + kb) : 0.f;   // warp-uniform address
            acc[c * 32 + j] = fmaf(__uint_as_float(v[j]), swv * sxv, acc[c * 32 + j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    if (ok && n < p.N) {
      if (p.splits == 1) {
        const float bv = p.bias ? p.bias[n] : 0.f;
#pragma unroll
        for (int j = 0; j < BT; ++j) {
          const int tok = tok0 + j;
          if (tok < p.M) p.D[(long long)tok * p.ldd + n] = __float2bfloat16(acc[j] + bv);
        }
      } else if (nkb > 0) {
#pragma unroll
        for (int j = 0; j < BT; ++j) {
          const int tok = tok0 + j;
          if (tok < p.M) atomicAdd(p.work + (long long)tok * p.N + n, acc[j]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TCOLS);
  }
}

__global__ void f8_finish_kernel(const float* __restrict__ work, const float* __restrict__ bias,
                                 __nv_bfloat16* __restrict__ D, long long ldd, int M, int N) {
  const long long n = (long long)M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int r = i / N, c = i % N;
    D[(long long)r * ldd + c] = __float2bfloat16(work[i] + (bias ? bias[c] : 0.f));
  }
}

template <int BT>
static int f8_launch(const F8Params& p, dim3 grid, cudaStream_t st) {
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_f8_kernel<BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<BT>::SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    set = true;
  }
  gemm_f8_kernel<BT><<<grid, F8_THREADS, F8Cfg<BT>::SMEM_BYTES, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

}  // namespace sx
using namespace sx;

// Grouped form: xq [rows, K] e4m3 expert-sorted rows (segments padded to 128), sx [rows, K/128];
// wq [E * N, K] e4m3, sw [E * N/128, K/128]; tile_group int32 [rows / 128]; out bf16 [rows, N]. N % 128 == 0.
extern "C" int sx_gemm_fp8_grouped(const void* xq, long long ldx, const float* sx_, const void* wq, long long ldw,
                                   const float* sw_, const int* tile_group, int num_experts, void* out, long long ldd,
                                   int rows, int N, int K, int* status, cudaStream_t st) {
  if (rows <= 0 || N <= 0) return 0;
  if (K % 128 || N % 128 || rows % 128 || (ldx % 16) || (ldw % 16) || !tile_group ||
      (reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return -1;
  F8Params p;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N * (uint64_t)num_experts};
    uint64_t strides[1] = {(uint64_t)ldw};
    uint32_t box[2] = {128, 128};
    int rc = make_tmap(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, wq, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows};
    uint64_t strides[1] = {(uint64_t)ldx};
    uint32_t box[2] = {128, 128};
    int rc = make_tmap(&p.tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, xq, dims, strides, box);
    if (rc) return rc;
  }
  p.sw = sw_; p.sx = sx_; p.bias = nullptr; p.D = (__nv_bfloat16*)out; p.work = nullptr; p.ldd = ldd;
  p.M = rows; p.N = N; p.K = K; p.kblks = K / 128; p.status = status; p.splits = 1; p.tile_group = tile_group;
  dim3 grid(N / 128, rows / 128, 1);
  return f8_launch<128>(p, grid, st);
}

// Bytes of fp32 workspace the call needs (0 when no split-K is used for this shape).
extern "C" long long sx_gemm_fp8_workspace(int M, int N, int K) {
  const int bt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  const long long ctas = (long long)((N + 127) / 128) * ((M + bt - 1) / bt);
  const int kblks = K / 128;
  int splits = (int)((148 * 2 + ctas - 1) / ctas);
  if (splits > kblks / 4) splits = kblks / 4;
  if (splits < 1) splits = 1;
  return splits > 1 ? (long long)M * N * 4 : 0;
}

// xq [M, K] e4m3 (ldx bytes per row), sx [M, K/128]; wq [N, K] e4m3 (ldw), sw [ceil(N/128), K/128]; out bf16 [M, N].
extern "C" int sx_gemm_fp8(const void* xq, long long ldx, const float* sx_, const void* wq, long long ldw, const float* sw_,
                           const float* bias, void* out, long long ldd, float* work, int M, int N, int K, int* status,
                           cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 128 || (ldx % 16) || (ldw % 16) || (reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return -1;
  F8Params p;
  const int bt = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t strides[1] = {(uint64_t)ldw};
    uint32_t box[2] = {128, 128};
    int rc = make_tmap(&p.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, wq, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t strides[1] = {(uint64_t)ldx};
    uint32_t box[2] = {128, (uint32_t)bt};
    int rc = make_tmap(&p.tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, xq, dims, strides, box);
    if (rc) return rc;
  }
  p.sw = sw_; p.sx = sx_; p.bias = bias; p.D = (__nv_bfloat16*)out; p.work = work; p.ldd = ldd;
  p.M = M; p.N = N; p.K = K; p.kblks = K / 128; p.status = status; p.tile_group = nullptr;
  const int nblks = (N + 127) / 128, tblks = (M + bt - 1) / bt;
  const long long ctas = (long long)nblks * tblks;
  int splits = (int)((148 * 2 + ctas - 1) / ctas);
  if (splits > p.kblks / 4) splits = p.kblks / 4;
  if (splits < 1) splits = 1;
  if (splits > 1 && !work) splits = 1;
  p.splits = splits;
  if (splits > 1) cudaMemsetAsync(work, 0, sizeof(float) * (size_t)M * N, st);
  dim3 grid(nblks, tblks, splits);
  int rc = bt == 32 ? f8_launch<32>(p, grid, st) : (bt == 64 ? f8_launch<64>(p, grid, st) : f8_launch<128>(p, grid, st));
  if (rc) return rc;
  if (splits > 1) {
    const long long n = (long long)M * N;
    const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
    f8_finish_kernel<<<blocks, 256, 0, st>>>(work, bias, (__nv_bfloat16*)out, ldd, M, N);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
