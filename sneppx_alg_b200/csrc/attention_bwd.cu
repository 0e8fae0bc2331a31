// A2: flash attention backward on tcgen05 (sm_100a), head_dim 128.
//
// One CTA owns 128 key/value rows of one (batch, kv head) and walks every query head of the GQA
// group and every 64-row query tile that can see those keys. Everything is computed transposed
// (key index on the TMEM lane axis), so that with the saved LSE no row reduction is needed:
//   S^T  = K Q^T            dP^T = V dO^T                         (128 x 64, fp32 in TMEM)
//   P^T  = exp2(S^T*c - LSE)    dS^T = P^T o (dP^T - delta) * scale  (registers -> bf16 smem tiles)
//   dV  += P^T dO           dK  += dS^T Q                          (128 x 128 accumulators in TMEM)
//   dQ^T = K^T dS^T         (128 x 64; staged through shared memory and added into dq_accum with bulk
//                            fp32 reductions, cp.reduce.async.bulk, one 4 KB slice per warp, off the critical path)
// The MN-major operand forms (dO, Q, K^T, dS^T as B/A operands) are read from the very tiles TMA
// brought or the softmax warps wrote; no transposed copy exists. dK/dV need no atomics because
// the whole GQA group is reduced inside the CTA.
// The reference only had a dQ kernel and a cuBLAS-composed backward that materialises P
// (kernel/cuda/attention_cuda.cu:388-492, kernel/cuda/autodiff_cuda.cu:746-862).
#include <limits.h>
#include "tc_common.cuh"
#include "common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int BWD_KV = 128;
constexpr int BWD_Q = 64;
constexpr int BWD_D = 128;
constexpr int BWD_THREADS = 320;  // TMA warp, MMA warp, 2 x 4 softmax-gradient warps (each group owns 32 query columns)

struct AttnBwdParams {
  CUtensorMap tmQ, tmK, tmV, tmdO;
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]
  float* dq_accum;     // [B, Sq, Hq, D] fp32
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long dk_row_stride, dv_row_stride, dk_batch_stride, dv_batch_stride;
  int* status;
  int B, Sq, Skv, Hq, Hk;
  int causal, window;
  float scale, scale_log2;
};

struct BwdCfg {
  static constexpr int KV_BYTES = BWD_KV * BWD_D * 2;  // 32 KB
  static constexpr int Q_BYTES = BWD_Q * BWD_D * 2;    // 16 KB
  static constexpr int PT_BYTES = BWD_KV * BWD_Q * 2;  // 16 KB
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_Q = 2 * KV_BYTES;             // 2 stages of (Q | dO)
  static constexpr int OFF_PT = OFF_Q + 2 * 2 * Q_BYTES;
  static constexpr int OFF_DST = OFF_PT + PT_BYTES;
  static constexpr int OFF_DQS = OFF_DST + PT_BYTES;     // dQ staging: 8 warps x [32 query rows][32 head-dim] fp32
  static constexpr int DQS_BYTES = BWD_Q * BWD_D * 4;    // 32 KB
  static constexpr int OFF_STAT = OFF_DQS + DQS_BYTES;   // spare
  static constexpr int OFF_BAR = OFF_STAT + 1024;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr uint32_t TM_S = 0, TM_DP = 64, TM_DQ = 128, TM_DV = 256, TM_DK = 384;
};

__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using Cfg = BwdCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sPT = smem + Cfg::OFF_PT;
  uint8_t* sDST = smem + Cfg::OFF_DST;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // [2]
  uint64_t* qdo_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;       // 1
  uint64_t* dp_full = bars + 6;      // 1
  uint64_t* pds_ready = bars + 7;    // 1 (8 arrivals)
  uint64_t* dq_full = bars + 8;      // 1
  uint64_t* dq_drained = bars + 9;   // 1 (8 arrivals): the dQ^T accumulator has been read out of TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heaviest key tiles first (under a causal mask tile 0 sees every query tile): kv head is the fastest block index.
  const int kv_tile = blockIdx.x / p.Hk, kv_head = blockIdx.x % p.Hk, b = blockIdx.z;
  const int G = p.Hq / p.Hk;
  const int kv0 = kv_tile * BWD_KV;
  const int offset = p.Skv - p.Sq;
  const int n_qt_total = (p.Sq + BWD_Q - 1) / BWD_Q;
  int qt_lo = 0, qt_hi = n_qt_total;  // [lo, hi)
  if (p.causal) {
    const int first_q = kv0 - offset;  // smallest query index that sees key kv0
    if (first_q > 0) qt_lo = first_q / BWD_Q;
  }
  if (p.window > 0) {
    const long long last_q = (long long)kv0 + BWD_KV - 1 + p.window - 1 - offset;
    if (last_q < 0) qt_hi = 0;
    else if (last_q / BWD_Q + 1 < qt_hi) qt_hi = (int)(last_q / BWD_Q + 1);
  }
  const int n_qt = max(qt_hi - qt_lo, 0);
  const int n_it = n_qt * G;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_ready, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, 8);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmQ);
    tma_prefetch_desc(&p.tmK);
    tma_prefetch_desc(&p.tmV);
    tma_prefetch_desc(&p.tmdO);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto tma5 = [](void* dst, const CUtensorMap* m, uint64_t* bar, int c1, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(0), "r"(c1), "r"(0),
        "r"(c3), "r"(c4)
        : "memory");
  };

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
      tma5(sK, &p.tmK, kv_full, kv0, kv_head, b);
      tma5(sV, &p.tmV, kv_full, kv0, kv_head, b);
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int head = kv_head * G + it / n_qt;
        const int qrow0 = (qt_lo + it % n_qt) * BWD_Q;
        if (!mbar_wait(&qdo_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&qdo_full[s], 2 * Cfg::Q_BYTES);
        tma5(sQ + s * 2 * Cfg::Q_BYTES, &p.tmQ, &qdo_full[s], qrow0, head, b);
        tma5(sQ + s * 2 * Cfg::Q_BYTES + Cfg::Q_BYTES, &p.tmdO, &qdo_full[s], qrow0, head, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, BWD_Q, 1, 0, 0);      // K Q^T, V dO^T
      constexpr uint32_t idesc_acc = umma_idesc_f16(128, BWD_D, 1, 0, 1);    // P^T dO, dS^T Q
      constexpr uint32_t idesc_dq = umma_idesc_f16(128, BWD_Q, 1, 1, 1);     // K^T dS^T
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aPT = smem_u32(sPT), aDST = smem_u32(sDST);
      auto issue_sdp = [&](int it) {
        const uint32_t q = smem_u32(sQ + (it & 1) * 2 * Cfg::Q_BYTES), dO = q + Cfg::Q_BYTES;
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_base + Cfg::TM_S, umma_desc_sw128(aK + c * 16384 + k * 32, 16, 1024),
                        umma_desc_sw128(q + c * 8192 + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(s_full);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_base + Cfg::TM_DP, umma_desc_sw128(aV + c * 16384 + k * 32, 16, 1024),
                        umma_desc_sw128(dO + c * 8192 + k * 32, 16, 1024), idesc_s, (c | k) ? 1u : 0u);
        umma_commit(dp_full);
      };
      bool ok = mbar_wait(kv_full, 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = mbar_wait(&qdo_full[0], 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_sdp(0);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait(pds_ready, it & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        if (it + 1 < n_it) {
          const int jn = it + 1;
          if (!mbar_wait(&qdo_full[jn & 1], (jn >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        }
        tc_fence_after();
        if (it + 1 < n_it) issue_sdp(it + 1);
        const uint32_t q = smem_u32(sQ + (it & 1) * 2 * Cfg::Q_BYTES), dO = q + Cfg::Q_BYTES;
        // dV += P^T dO ; dK += dS^T Q   (K = 64 query rows: 4 k-steps)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ss(tmem_base + Cfg::TM_DV, umma_desc_sw128(aPT + k * 32, 16, 1024),
                      umma_desc_sw128(dO + k * 2048, 8192, 1024), idesc_acc, (it | k) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ss(tmem_base + Cfg::TM_DK, umma_desc_sw128(aDST + k * 32, 16, 1024),
                      umma_desc_sw128(q + k * 2048, 8192, 1024), idesc_acc, (it | k) ? 1u : 0u);
        // dQ^T = K^T dS^T  (K = 128 key rows: 8 k-steps); the accumulator of the previous iteration must be read out
        if (it > 0) {
          if (!mbar_wait(dq_drained, (it - 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ss(tmem_base + Cfg::TM_DQ, umma_desc_sw128(aK + k * 2048, 16384, 1024),
                      umma_desc_sw128(aDST + k * 2048, 16384, 1024), idesc_dq, k ? 1u : 0u);
        umma_commit(&qdo_empty[it & 1]);
        umma_commit(dq_full);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax-gradient warps
    const int wg = (warp - 2) >> 2;     // column group: query columns [32*wg, 32*wg + 32) of the tile
    const int qd = warp & 3;
    const int r = qd * 32 + lane;       // key row inside the tile == TMEM lane
    const int kv_idx = kv0 + r;
    const int c0 = wg * 32;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    bool ok = n_it > 0;
    float* stage = reinterpret_cast<float*>(smem + Cfg::OFF_DQS) + (warp - 2) * 1024;  // this warp's [32 q][32 d] slice
    auto drain_dq = [&](int it) {
      // dQ^T tile: lane = head-dim index, column = query row. dq_accum is tiled so that every warp's slice is one
      // contiguous 4 KB run: [b][head][q tile][column group][lane quarter][32 query rows][32 head-dim].
      const int head = kv_head * G + it / n_qt;
      const int qt = qt_lo + it % n_qt;
      float* dst = p.dq_accum + (((((long long)b * p.Hq + head) * n_qt_total + qt) * 2 + wg) * 4 + qd) * 1024;
      uint32_t v[32];
      tmem_ld32(tmem_base + Cfg::TM_DQ + lane_addr + c0, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(dq_drained);
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the previous reduction has read the slice
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 32; ++i) stage[i * 32 + lane] = __uint_as_float(v[i]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
                     "r"(smem_u32(stage)), "r"(4096)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    };
    for (int it = 0; it < n_it && ok; ++it) {
      const int head = kv_head * G + it / n_qt;
      const int qrow0 = (qt_lo + it % n_qt) * BWD_Q;
      // lane i keeps LSE / delta of query column c0 + i; columns are broadcast by shuffle
      const int qi_l = qrow0 + c0 + lane;
      const long long so = ((long long)b * p.Hq + head) * p.Sq + qi_l;
      const float lse_r = qi_l < p.Sq ? p.lse[so] * 1.4426950408889634f : INFINITY;
      const float dl_r = qi_l < p.Sq ? p.delta[so] : 0.f;
      const bool need_mask = (p.causal && kv0 + BWD_KV - 1 > qrow0 + offset) || (kv0 + BWD_KV > p.Skv) ||
                             (p.window > 0 && kv0 < qrow0 + BWD_Q - 1 + offset - p.window + 1);
      uint32_t pt[16];
      uint32_t ds[16];
      if (!mbar_wait_warp(s_full, it & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v[32];
        tmem_ld32(tmem_base + Cfg::TM_S + lane_addr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(__uint_as_float(v[i]) * p.scale_log2 - __shfl_sync(0xffffffffu, lse_r, i));
          float p1 = exp2f(__uint_as_float(v[i + 1]) * p.scale_log2 - __shfl_sync(0xffffffffu, lse_r, i + 1));
          if (need_mask) {
            const int q0i = qrow0 + c0 + i + offset;
            if (kv_idx > q0i && p.causal) p0 = 0.f;
            if (kv_idx > q0i + 1 && p.causal) p1 = 0.f;
            if (p.window > 0) {
              if (kv_idx < q0i - p.window + 1) p0 = 0.f;
              if (kv_idx < q0i + 1 - p.window + 1) p1 = 0.f;
            }
            if (kv_idx >= p.Skv) { p0 = 0.f; p1 = 0.f; }
          }
          pt[i / 2] = pack_bf16x2(p0, p1);
        }
      }
      if (!mbar_wait_warp(dp_full, it & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v[32];
        tmem_ld32(tmem_base + Cfg::TM_DP + lane_addr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float pl = __uint_as_float(pt[i / 2] << 16), ph = __uint_as_float(pt[i / 2] & 0xffff0000u);
          const float d0 = pl * (__uint_as_float(v[i]) - __shfl_sync(0xffffffffu, dl_r, i)) * p.scale;
          const float d1 = ph * (__uint_as_float(v[i + 1]) - __shfl_sync(0xffffffffu, dl_r, i + 1)) * p.scale;
          ds[i / 2] = pack_bf16x2(d0, d1);
        }
      }
      // the P^T / dS^T tiles are free, and dQ^T of iteration it-1 is complete, once iteration it-1 has fully executed
      if (it > 0) {
        if (!mbar_wait_warp(dq_full, (it - 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int cc = wg * 4 + k;
        const int off = r * 128 + ((cc ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(sPT + off) = make_uint4(pt[k * 4], pt[k * 4 + 1], pt[k * 4 + 2], pt[k * 4 + 3]);
        *reinterpret_cast<uint4*>(sDST + off) = make_uint4(ds[k * 4], ds[k * 4 + 1], ds[k * 4 + 2], ds[k * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
      if (it > 0) drain_dq(it - 1);  // overlaps the S / dP / dV / dK MMAs the arrive above released
    }
    if (lane == 0 && !ok) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (ok && n_it > 0) {
      if (mbar_wait_warp(dq_full, (n_it - 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) {
        tc_fence_after();
        drain_dq(n_it - 1);
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        // dK / dV accumulators -> bf16 rows
        const bool row_ok = kv_idx < p.Skv;
        __nv_bfloat16* dkr = p.dK + (long long)b * p.dk_batch_stride + (long long)kv_idx * p.dk_row_stride +
                             (long long)kv_head * BWD_D;
        __nv_bfloat16* dvr = p.dV + (long long)b * p.dv_batch_stride + (long long)kv_idx * p.dv_row_stride +
                             (long long)kv_head * BWD_D;
#pragma unroll 1
        for (int which = wg; which <= wg; ++which) {  // group 0 stores dV, group 1 stores dK
          const uint32_t src = tmem_base + (which ? Cfg::TM_DK : Cfg::TM_DV) + lane_addr;
          __nv_bfloat16* dst = which ? dkr : dvr;
#pragma unroll 1
          for (int c = 0; c < BWD_D / 32; ++c) {
            uint32_t v[32];
            tmem_ld32(src + c * 32, v);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                o.y = pack_bf16x2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                o.z = pack_bf16x2(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                o.w = pack_bf16x2(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                *reinterpret_cast<uint4*>(dst + c * 32 + i) = o;
              }
            }
          }
        }
      }
    } else if (n_it == 0) {
      if (kv_idx < p.Skv) {
        __nv_bfloat16* dkr = p.dK + (long long)b * p.dk_batch_stride + (long long)kv_idx * p.dk_row_stride +
                             (long long)kv_head * BWD_D;
        __nv_bfloat16* dvr = p.dV + (long long)b * p.dv_batch_stride + (long long)kv_idx * p.dv_row_stride +
                             (long long)kv_head * BWD_D;
        for (int i = 0; i < BWD_D; i += 8) {
          *reinterpret_cast<uint4*>(dkr + i) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dvr + i) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d dO * O ; one warp per (token, head).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                  float* __restrict__ delta, int B, int S, int H, int D, long long do_row_stride,
                                  long long o_row_stride) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * S * H) return;
  const int h = w % H;
  const long long tok = w / H;  // b*S + s
  const __nv_bfloat16* a = dO + tok * do_row_stride + (long long)h * D;
  const __nv_bfloat16* c = O + tok * o_row_stride + (long long)h * D;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(c + i));
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  if (lane == 0) {
    const long long bb = tok / S, ss = tok % S;
    delta[(bb * H + h) * S + ss] = s;
  }
}

// dq_accum (tiled as the backward kernel writes it) -> bf16 dQ rows. One thread converts 4 head-dim values.
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dQ, int B, int Sq,
                                       int Hq, long long dq_row_stride) {
  const int n_qt = (Sq + BWD_Q - 1) / BWD_Q;
  const long long n = (long long)B * Hq * n_qt * (BWD_Q * BWD_D / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    // i enumerates float4 groups of the tiled buffer in storage order
    const int di4 = i & 7;                 // 8 float4 per 32-wide head-dim run
    const int qi = (i >> 3) & 31;
    const int qd = (i >> 8) & 3;
    const int wg = (i >> 10) & 1;
    const long long t = i >> 11;           // (b * Hq + head) * n_qt + tile
    const int tile = t % n_qt;
    const long long bh = t / n_qt;
    const int head = bh % Hq;
    const long long bb = bh / Hq;
    const int srow = tile * BWD_Q + wg * 32 + qi;
    if (srow >= Sq) continue;
    const float4 v = *reinterpret_cast<const float4*>(acc + i * 4);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dQ + (bb * Sq + srow) * dq_row_stride + (long long)head * BWD_D + qd * 32 + di4 * 4) = o;
  }
}

static int make_attn_map_bwd(CUtensorMap* tm, const void* base, int B, int S, int H, int D, long long row_stride,
                             long long batch_stride, int box_rows) {
  uint64_t dims[5] = {64, (uint64_t)S, (uint64_t)(D / 64), (uint64_t)H, (uint64_t)B};
  uint64_t strides[4] = {(uint64_t)row_stride * 2, 128, (uint64_t)D * 2, (uint64_t)batch_stride * 2};
  uint32_t box[5] = {64, (uint32_t)box_rows, (uint32_t)(D / 64), 1, 1};
  return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, box);
}

}  // namespace sx
using namespace sx;

// Requirements: D == 128, v_head_div == 1, dQ batch stride == Sq * dq_row_stride; dq_accum holds
// B * Hq * ceil(Sq / 64) * 64 * 128 floats.
extern "C" int sx_attn_bwd(const SxAttnArgs* a, cudaStream_t st) {
  if (a->D != BWD_D) return -1;
  if (a->Hq % a->Hk) return -2;
  if (a->v_head_div > 1) return -4;
  if ((a->q_row_stride % 8) || (a->k_row_stride % 8) || (a->v_row_stride % 8) || (a->do_row_stride % 8) ||
      (a->dq_row_stride % 4) || (a->dk_row_stride % 8) || (a->dv_row_stride % 8))
    return -3;
  AttnBwdParams p;
  int rc = make_attn_map_bwd(&p.tmQ, a->Q, a->B, a->Sq, a->Hq, a->D, a->q_row_stride, a->q_batch_stride, BWD_Q);
  if (rc) return rc;
  rc = make_attn_map_bwd(&p.tmdO, a->dO, a->B, a->Sq, a->Hq, a->D, a->do_row_stride, (long long)a->Sq * a->do_row_stride,
                         BWD_Q);
  if (rc) return rc;
  rc = make_attn_map_bwd(&p.tmK, a->K, a->B, a->Skv, a->Hk, a->D, a->k_row_stride, a->k_batch_stride, BWD_KV);
  if (rc) return rc;
  rc = make_attn_map_bwd(&p.tmV, a->V, a->B, a->Skv, a->Hk, a->D, a->v_row_stride, a->v_batch_stride, BWD_KV);
  if (rc) return rc;
  const long long tokens = (long long)a->B * a->Sq;
  const int n_qt = (a->Sq + BWD_Q - 1) / BWD_Q;
  // dq_accum holds whole 64-row query tiles: B * Hq * n_qt * 64 * 128 floats
  const long long acc_floats = (long long)a->B * a->Hq * n_qt * BWD_Q * BWD_D;
  cudaMemsetAsync(a->dq_accum, 0, sizeof(float) * acc_floats, st);
  {
    const long long warps = tokens * a->Hq;
    const int blocks = (int)((warps * 32 + 255) / 256);
    attn_delta_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)a->dO, (const __nv_bfloat16*)a->O, a->delta, a->B,
                                              a->Sq, a->Hq, a->D, a->do_row_stride, a->o_row_stride);
  }
  p.lse = a->lse; p.delta = a->delta; p.dq_accum = a->dq_accum;
  p.dK = (__nv_bfloat16*)a->dK; p.dV = (__nv_bfloat16*)a->dV;
  p.dk_row_stride = a->dk_row_stride; p.dv_row_stride = a->dv_row_stride;
  p.dk_batch_stride = a->dk_batch_stride; p.dv_batch_stride = a->dv_batch_stride;
  p.status = a->status;
  p.B = a->B; p.Sq = a->Sq; p.Skv = a->Skv; p.Hq = a->Hq; p.Hk = a->Hk;
  p.causal = a->causal; p.window = a->window;
  p.scale = a->scale; p.scale_log2 = a->scale * 1.4426950408889634f;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg::SMEM_BYTES) !=
        cudaSuccess)
      return -10;
    set = true;
  }
  dim3 grid(((a->Skv + BWD_KV - 1) / BWD_KV) * a->Hk, 1, a->B);
  attn_bwd_kernel<<<grid, BWD_THREADS, BwdCfg::SMEM_BYTES, st>>>(p);
  {
    const long long n = acc_floats / 4;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    attn_dq_convert_kernel<<<blocks, 256, 0, st>>>(a->dq_accum, (__nv_bfloat16*)a->dQ, a->B, a->Sq, a->Hq,
                                                   a->dq_row_stride);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
