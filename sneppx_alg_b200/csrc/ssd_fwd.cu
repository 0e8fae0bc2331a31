// S1: the output stage of the chunked SSD scan as one tcgen05 kernel (sm_100a), chunk 128, state 128, headdim 64.
//
// One CTA owns one (batch, chunk, B/C group) and walks the heads h of that group:
//   G     = C B^T                                 tcgen05.mma SS once per CTA, fp32 in TMEM (shared by the heads)
//   M_h   = G o exp(cs_l - cs_s) dt_s [s <= l]    one chunk row per thread (TMEM lane == row), written back to TMEM
//                                                 as packed bf16
//   Yi_h  = M_h X_h                               tcgen05.mma TS: M straight from TMEM, X consumed MN-major from its
//                                                 [token, headdim] tile
//   Yo_h  = C Hprev_h^T                           tcgen05.mma SS, Hprev = the state entering the chunk
//   y_h   = Yi_h + exp(cs_l) Yo_h + D_h x_h       epilogue of the same four warps
// C, B and x are read in place from their token-major tensors (TMA, token stride given), so neither the
// heads-first copies nor any Q x Q matrix ever reaches HBM. tcgen05.mma executes in issue order: the convert
// warps only overwrite M after the MMAs of the previous head have signalled y_full.
// Every wait is bounded (status word + early exit), TMEM is freed on every path.
// The reference has no such kernel: its selective scan is serial over the sequence
// (algorithms/hss/cuda/hss_cuda_extended.cu:27-77) and its Mamba-2 block is a stub (kernel/arch/mamba2.c:36-133).
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int SF_Q = 128;   // chunk length == MMA M
constexpr int SF_N = 128;   // state size
constexpr int SF_P = 64;    // head dimension
constexpr int SF_THREADS = 192;   // TMA warp, MMA warp, 4 convert / epilogue warps

struct SsdFwdParams {
  CUtensorMap tmC, tmB, tmX, tmH;
  const float* cs;     // [BC, H, Q] inclusive cumulative sum of dt * A inside the chunk
  const float* dt;     // [BC, H, Q]
  const float* D;      // [H] or null
  const __nv_bfloat16* x;   // token-major [tokens, H, P], token stride x_ld
  __nv_bfloat16* y;         // token-major [tokens, H, P] contiguous
  int* status;
  long long x_ld;
  int H, G;
};

struct SsdFwdCfg {
  static constexpr int CB_BYTES = SF_Q * SF_N * 2;      // 32 KB: C or B chunk, two 64-column slabs
  static constexpr int X_BYTES = SF_Q * SF_P * 2;       // 16 KB
  static constexpr int H_BYTES = SF_P * SF_N * 2;       // 16 KB: two slabs of [64 x 64]
  static constexpr int OFF_B = CB_BYTES;
  static constexpr int OFF_X = 2 * CB_BYTES;
  static constexpr int OFF_H = OFF_X + 2 * X_BYTES;
  static constexpr int OFF_VEC = OFF_H + 2 * H_BYTES;   // cs[128], dt[128] floats
  static constexpr int OFF_BAR = OFF_VEC + 1024;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // TMEM columns: G 0..127, M (packed bf16) 128..191, Yi 192..255, Yo 256..319
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_M = 128, COL_YI = 192, COL_YO = 256;
};

__global__ void __launch_bounds__(SF_THREADS, 1) ssd_chunk_fwd_kernel(const __grid_constant__ SsdFwdParams p) {
  using Cfg = SsdFwdCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sC = smem;
  uint8_t* sB = smem + Cfg::OFF_B;
  uint8_t* sX = smem + Cfg::OFF_X;
  uint8_t* sH = smem + Cfg::OFF_H;
  float* s_cs = reinterpret_cast<float*>(smem + Cfg::OFF_VEC);
  float* s_dt = s_cs + SF_Q;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* cb_full = bars;          // 1
  uint64_t* xh_full = bars + 1;      // [2]
  uint64_t* xh_empty = bars + 3;     // [2]
  uint64_t* g_full = bars + 5;       // 1
  uint64_t* m_full = bars + 6;       // 1 (4 arrivals)
  uint64_t* y_full = bars + 7;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x;
  const long long bc = blockIdx.y;
  const int rep = p.H / p.G;
  const int t0 = (int)(bc * SF_Q);   // first token of the chunk

  if (threadIdx.x == 0) {
    mbar_init(cb_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&xh_full[i], 1);
      mbar_init(&xh_empty[i], 1);
    }
    mbar_init(g_full, 1);
    mbar_init(m_full, 4);
    mbar_init(y_full, 1);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmC);
    tma_prefetch_desc(&p.tmB);
    tma_prefetch_desc(&p.tmX);
    tma_prefetch_desc(&p.tmH);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(cb_full, 2 * Cfg::CB_BYTES);
      tma_load_4d(sC, &p.tmC, cb_full, 0, t0, 0, g);
      tma_load_4d(sB, &p.tmB, cb_full, 0, t0, 0, g);
      for (int i = 0; i < rep; ++i) {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int h = g * rep + i;
        if (!mbar_wait(&xh_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&xh_full[s], Cfg::X_BYTES + Cfg::H_BYTES);
        tma_load_3d(sX + s * Cfg::X_BYTES, &p.tmX, &xh_full[s], 0, t0, h);
        tma_load_3d(sH + s * Cfg::H_BYTES, &p.tmH, &xh_full[s], 0, (int)((bc * p.H + h) * SF_P), 0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_g = umma_idesc_f16(SF_Q, SF_Q, 1, 0, 0);      // C B^T, both K-major
      constexpr uint32_t idesc_mx = umma_idesc_f16(SF_Q, SF_P, 1, 0, 1);     // M (TMEM) x X (MN-major)
      constexpr uint32_t idesc_yo = umma_idesc_f16(SF_Q, SF_P, 1, 0, 0);     // C x Hprev^T, both K-major
      bool ok = mbar_wait(cb_full, 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        const uint32_t a0 = smem_u32(sC), b0 = smem_u32(sB);
#pragma unroll
        for (int c = 0; c < SF_N / 64; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_base, umma_desc_sw128(a0 + c * (SF_Q * 128) + k * 32, 16, 1024),
                        umma_desc_sw128(b0 + c * (SF_Q * 128) + k * 32, 16, 1024), idesc_g, (c | k) ? 1u : 0u);
        umma_commit(g_full);
      }
      for (int i = 0; i < rep && ok; ++i) {
        const int s = i & 1;
        if (!mbar_wait(&xh_full[s], (i >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        if (!mbar_wait(m_full, i & 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t xb = smem_u32(sX + s * Cfg::X_BYTES), hb = smem_u32(sH + s * Cfg::H_BYTES);
        const uint32_t a0 = smem_u32(sC);
#pragma unroll
        for (int k = 0; k < SF_Q / 16; ++k)
          umma_f16_ts(tmem_base + Cfg::COL_YI, tmem_base + Cfg::COL_M + k * 8,
                      umma_desc_sw128(xb + k * 2048, SF_Q * 128, 1024), idesc_mx, k ? 1u : 0u);
#pragma unroll
        for (int c = 0; c < SF_N / 64; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_base + Cfg::COL_YO, umma_desc_sw128(a0 + c * (SF_Q * 128) + k * 32, 16, 1024),
                        umma_desc_sw128(hb + c * (SF_P * 128) + k * 32, 16, 1024), idesc_yo, (c | k) ? 1u : 0u);
        umma_commit(y_full);
        umma_commit(&xh_empty[s]);
      }
    }
  } else {
    // ------------------------------------------------------------ convert + epilogue warps (one chunk row each)
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    const uint32_t tG = tmem_base + lane_addr;
    const uint32_t tM = tG + Cfg::COL_M, tYi = tG + Cfg::COL_YI, tYo = tG + Cfg::COL_YO;
    bool ok = mbar_wait_warp(g_full, 0, s_abort, p.status, ST_TIMEOUT_CONVERT);
    tc_fence_after();
    // The loop always runs all heads and both named barriers, also after a wait gave up (`ok` false): the 128 threads
    // must reach bar.sync the same number of times or the CTA would never finish.
    for (int i = 0; i < rep; ++i) {
      const int h = g * rep + i;
      const long long vec = (bc * p.H + h) * SF_Q;
      const float cs_l = p.cs[vec + row];
      asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone is done with the previous head's vectors
      s_cs[row] = cs_l;
      s_dt[row] = p.dt[vec + row];
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!ok) continue;
      uint32_t pk[SF_Q / 2];
#pragma unroll
      for (int c = 0; c < SF_Q / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tG + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int s0 = c * 32 + j;
          const float v0 = s0 <= row ? __uint_as_float(r[j]) * __expf(cs_l - s_cs[s0]) * s_dt[s0] : 0.f;
          const float v1 = s0 + 1 <= row ? __uint_as_float(r[j + 1]) * __expf(cs_l - s_cs[s0 + 1]) * s_dt[s0 + 1] : 0.f;
          pk[(c * 32 + j) >> 1] = pack_bf16x2(v0, v1);
        }
      }
      tmem_st32(tM, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st32(tM + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(m_full);
      // ---- epilogue of this head
      if (!mbar_wait_warp(y_full, i & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; continue; }
      tc_fence_after();
      const float e = __expf(cs_l);
      const float dh = p.D ? p.D[h] : 0.f;
      const long long tok = (long long)t0 + row;
      const __nv_bfloat16* xrow = p.x + tok * p.x_ld + (long long)h * SF_P;
      __nv_bfloat16* yrow = p.y + (tok * p.H + h) * SF_P;
#pragma unroll
      for (int c = 0; c < SF_P / 32; ++c) {
        uint32_t a[32], b[32];
        tmem_ld32(tYi + c * 32, a);
        tmem_ld32(tYo + c * 32, b);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          const uint4 xr = *reinterpret_cast<const uint4*>(xrow + c * 32 + j);
          const uint32_t xw[4] = {xr.x, xr.y, xr.z, xr.w};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float x0 = __uint_as_float(xw[q] << 16), x1 = __uint_as_float(xw[q] & 0xffff0000u);
            const float y0 = __uint_as_float(a[j + 2 * q]) + e * __uint_as_float(b[j + 2 * q]) + dh * x0;
            const float y1 = __uint_as_float(a[j + 2 * q + 1]) + e * __uint_as_float(b[j + 2 * q + 1]) + dh * x1;
            o[q] = pack_bf16x2(y0, y1);
          }
          *reinterpret_cast<uint4*>(yrow + c * 32 + j) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
      tc_fence_before();   // the next head's MMAs overwrite Yi / Yo only after these reads
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace sx
using namespace sx;

// C, B: token-major [tokens, G, 128] bf16 with token stride c_ld / b_ld (elements); x: [tokens, H, 64], token stride
// x_ld; Hprev: [BC, H, 64, 128] bf16 contiguous; cs, dt: [BC, H, 128] fp32; y: [tokens, H, 64] bf16 contiguous.
// tokens = BC * 128.
extern "C" int sx_ssd_chunk_fwd(const void* C, long long c_ld, const void* B, long long b_ld, const void* x,
                                long long x_ld, const void* Hprev, const void* cs, const void* dt, const void* D,
                                void* y, long long BC, int H, int G, int* status, cudaStream_t st) {
  if (H % G || BC <= 0 || BC > 65535 || (c_ld % 8) || (b_ld % 8) || (x_ld % 8)) return -1;
  const long long tokens = BC * SF_Q;
  if (tokens * 1ll > 0x7fffffffll || BC * H * SF_P > 0x7fffffffll) return -2;
  SsdFwdParams p;
  {
    uint64_t dims[4] = {64, (uint64_t)tokens, SF_N / 64, (uint64_t)G};
    uint64_t sc[3] = {(uint64_t)c_ld * 2, 128, (uint64_t)SF_N * 2};
    uint64_t sb[3] = {(uint64_t)b_ld * 2, 128, (uint64_t)SF_N * 2};
    uint32_t box[4] = {64, SF_Q, SF_N / 64, 1};
    int rc = make_tmap(&p.tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, C, dims, sc, box);
    if (rc) return rc;
    rc = make_tmap(&p.tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, B, dims, sb, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {64, (uint64_t)tokens, (uint64_t)H};
    uint64_t strides[2] = {(uint64_t)x_ld * 2, (uint64_t)SF_P * 2};
    uint32_t box[3] = {64, SF_Q, 1};
    const int rc = make_tmap(&p.tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, x, dims, strides, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {64, (uint64_t)(BC * H * SF_P), SF_N / 64};
    uint64_t strides[2] = {(uint64_t)SF_N * 2, 128};
    uint32_t box[3] = {64, SF_P, SF_N / 64};
    const int rc = make_tmap(&p.tmH, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, Hprev, dims, strides, box);
    if (rc) return rc;
  }
  p.cs = (const float*)cs;
  p.dt = (const float*)dt;
  p.D = (const float*)D;
  p.x = (const __nv_bfloat16*)x;
  p.y = (__nv_bfloat16*)y;
  p.status = status;
  p.x_ld = x_ld;
  p.H = H;
  p.G = G;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(ssd_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SsdFwdCfg::SMEM_BYTES) != cudaSuccess) return -10;
    set = true;
  }
  ssd_chunk_fwd_kernel<<<dim3(G, (unsigned)BC), SF_THREADS, SsdFwdCfg::SMEM_BYTES, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
