// Q2: dequant-GEMM on tcgen05. Y[M, N] = X[M, K] (bf16) x dequant(W)[N, K]^T with W stored as
//   fp8 e4m3 + fp32 scales per 128 x 128 block, or INT4 (two per byte, offset 8) + fp32 scales per (row, 128 columns).
// The weight tile never exists in bf16 in global memory: four converter warps read the packed tile with 16-byte
// loads (next stage prefetched into registers while the current one is converted), scale and write bf16 straight
// into the 128-byte-swizzled K-major smem tile the MMA consumes; activations arrive by TMA. The HBM traffic of a
// decode step is therefore the quantised weights only.
// Structure (320 threads): warp 0 TMA producer (A), warp 1 MMA issuer, warps 2-5 converters (B), warps 6-9 epilogue.
// The reference has quantise / dequantise kernels only (kernel/quantization/quantize_cuda.cu), no GEMM on them.
#include <cuda_fp8.h>
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int DQ_BM = 128, DQ_BN = 128, DQ_BK = 64, DQ_STAGES = 6, DQ_THREADS = 320;
constexpr int DQ_A_BYTES = DQ_BM * DQ_BK * 2, DQ_B_BYTES = DQ_BN * DQ_BK * 2;
constexpr int DQ_STAGE_BYTES = DQ_A_BYTES + DQ_B_BYTES;
constexpr int DQ_SMEM = DQ_STAGES * DQ_STAGE_BYTES + 1024 + 512;

struct DqParams {
  CUtensorMap tmA;
  const uint8_t* W;       // fp8: [N, K] bytes; int4: [N, K/2] bytes
  const float* scales;    // fp8: [ceil(N/128), ceil(K/128)]; int4: [N, K/128]
  const float* bias;
  __nv_bfloat16* D;
  long long ldd;
  int M, N, K, mode;      // mode 0 fp8 e4m3, 1 int4
  int m_blks, n_blks;
  int* status;
};

__device__ __forceinline__ float e4m3_to_f(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__global__ void __launch_bounds__(DQ_THREADS, 1) gemm_dq_kernel(const __grid_constant__ DqParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DQ_STAGES * DQ_STAGE_BYTES);
  uint64_t* a_full = bars;                    // [STAGES] TMA
  uint64_t* b_full = bars + DQ_STAGES;        // [STAGES] 4 converter warps
  uint64_t* empty = bars + 2 * DQ_STAGES;     // [STAGES] MMA commit
  uint64_t* tfull = bars + 3 * DQ_STAGES;     // [2]
  uint64_t* tempty = tfull + 2;               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < DQ_STAGES; ++s) {
      mbar_init(&a_full[s], 1);
      mbar_init(&b_full[s], 4);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmA);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * DQ_BN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total = p.m_blks * p.n_blks;
  const int num_kb = (p.K + DQ_BK - 1) / DQ_BK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int m_blk = t % p.m_blks;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(&a_full[stage], DQ_A_BYTES);
          tma_load_3d(smem + stage * DQ_STAGE_BYTES, &p.tmA, &a_full[stage], kb * DQ_BK, m_blk * DQ_BM, 0);
          if (++stage == DQ_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(DQ_BM, DQ_BN, 1, 0, 0);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const int acc = it & 1;
        if (!mbar_wait(&tempty[acc], ((it >> 1) & 1) ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&a_full[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA) ||
              !mbar_wait(&b_full[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * DQ_STAGE_BYTES), sb = sa + DQ_A_BYTES;
#pragma unroll
          for (int k = 0; k < DQ_BK / 16; ++k)
            umma_f16_ss(tmem_base + acc * DQ_BN, umma_desc_sw128(sa + k * 32, 16, 1024),
                        umma_desc_sw128(sb + k * 32, 16, 1024), idesc, (kb | k) ? 1u : 0u);
          umma_commit(&empty[stage]);
          if (++stage == DQ_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull[acc]);
        ++it;
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ converters: 128 threads, one weight row each
    const int r = (warp - 2) * 32 + lane;  // row inside the N tile
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const int kb128 = (p.K + 127) / 128;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const int n_blk = t / p.m_blks;
      const int n = n_blk * DQ_BN + r;
      const bool row_ok = n < p.N;
      // prefetch registers for the first k block
      uint4 raw[4];
      auto fetch = [&](int kb) {
        if (!row_ok) return;
        if (p.mode == 0) {
          const uint8_t* src = p.W + (long long)n * p.K + kb * DQ_BK;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            raw[i] = (kb * DQ_BK + i * 16 < p.K) ? *reinterpret_cast<const uint4*>(src + i * 16) : make_uint4(0, 0, 0, 0);
        } else {
          const uint8_t* src = p.W + (long long)n * (p.K / 2) + kb * (DQ_BK / 2);
#pragma unroll
          for (int i = 0; i < 2; ++i)
            raw[i] = (kb * DQ_BK + i * 32 < p.K) ? *reinterpret_cast<const uint4*>(src + i * 16) : make_uint4(0, 0, 0, 0);
        }
      };
      fetch(0);
      for (int kb = 0; kb < num_kb; ++kb) {
        uint4 cur[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) cur[i] = raw[i];
        if (kb + 1 < num_kb) fetch(kb + 1);
        float sc = 0.f;
        if (row_ok)
          sc = p.mode == 0 ? p.scales[(long long)(n / 128) * kb128 + (kb * DQ_BK) / 128]
                           : p.scales[(long long)n * (p.K / 128) + (kb * DQ_BK) / 128];
        if (!mbar_wait_warp(&empty[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_CONVERT)) { ok = false; break; }
        uint8_t* sb = smem + stage * DQ_STAGE_BYTES + DQ_A_BYTES + r * 128;
        if (p.mode == 0) {
          const uint8_t* b8 = reinterpret_cast<const uint8_t*>(cur);
#pragma unroll
          for (int c = 0; c < 8; ++c) {  // 8 chunks of 8 bf16
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              ow[j] = row_ok ? pack_bf16x2(e4m3_to_f(b8[c * 8 + 2 * j]) * sc, e4m3_to_f(b8[c * 8 + 2 * j + 1]) * sc) : 0u;
            *reinterpret_cast<uint4*>(sb + ((c ^ (r & 7)) << 4)) = o;
          }
        } else {
          const uint8_t* b4 = reinterpret_cast<const uint8_t*>(cur);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint8_t by = b4[c * 4 + j];
              ow[j] = row_ok ? pack_bf16x2(((int)(by & 15) - 8) * sc, ((int)(by >> 4) - 8) * sc) : 0u;
            }
            *reinterpret_cast<uint4*>(sb + ((c ^ (r & 7)) << 4)) = o;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&b_full[stage]);
        if (++stage == DQ_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;
    int it = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x) {
      const int m_blk = t % p.m_blks, n_blk = t / p.m_blks;
      const int acc = it & 1;
      if (!mbar_wait_warp(&tfull[acc], (it >> 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m_blk * DQ_BM + q * 32 + lane;
#pragma unroll 1
      for (int c = 0; c < DQ_BN / 32; ++c) {
        const int col0 = n_blk * DQ_BN + c * 32;
        if (col0 >= p.N) break;
        uint32_t v[32];
        tmem_ld32(tmem_base + acc * DQ_BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), v);
        tmem_ld_wait();
        if (row >= p.M) continue;
        __nv_bfloat16* dp = p.D + (long long)row * p.ldd + col0;
        const bool full = col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0);
        if (full) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[j + i]) + (p.bias ? p.bias[col0 + j + i] : 0.f);
            uint4 o;
            o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
            o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(dp + j) = o;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) dp[j] = __float2bfloat16(__uint_as_float(v[j]) + (p.bias ? p.bias[col0 + j] : 0.f));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      ++it;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * DQ_BN);
  }
}

}  // namespace sx
using namespace sx;

// X: bf16 [M, K] (ldx); W packed (mode 0: fp8 e4m3 [N, K], mode 1: int4 [N, K/2]); D: bf16 [M, N] (ldd).
extern "C" int sx_gemm_dequant(const void* X, long long ldx, const void* W, const float* scales, const float* bias,
                               void* D, long long ldd, int M, int N, int K, int mode, int* status, cudaStream_t st) {
  if (K % 128 || ldx % 8 || (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return -1;
  if (M <= 0 || N <= 0) return 0;
  DqParams p;
  uint64_t dims[3] = {(uint64_t)K, (uint64_t)M, 1};
  uint64_t strides[2] = {(uint64_t)ldx * 2, (uint64_t)M * ldx * 2};
  uint32_t box[3] = {DQ_BK, DQ_BM, 1};
  int rc = make_tmap(&p.tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, X, dims, strides, box);
  if (rc) return rc;
  p.W = (const uint8_t*)W; p.scales = scales; p.bias = bias; p.D = (__nv_bfloat16*)D; p.ldd = ldd;
  p.M = M; p.N = N; p.K = K; p.mode = mode;
  p.m_blks = (M + DQ_BM - 1) / DQ_BM; p.n_blks = (N + DQ_BN - 1) / DQ_BN;
  p.status = status;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(gemm_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM) != cudaSuccess) return -10;
    set = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = p.m_blks * p.n_blks;
  gemm_dq_kernel<<<tiles < sms ? tiles : sms, DQ_THREADS, DQ_SMEM, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
