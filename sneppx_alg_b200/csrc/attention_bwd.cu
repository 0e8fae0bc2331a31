// A2: flash attention backward on tcgen05 (sm_100a), head_dim 128.
//
// One CTA owns 128 key/value rows of one (batch, kv head) and walks every query head of the GQA
// group and every 64-row query tile that can see those keys. Everything is computed transposed
// (key index on the TMEM lane axis), so that with the saved LSE no row reduction is needed:
//   S^T  = K Q^T            dP^T = V dO^T                         (128 x 64, fp32 in TMEM)
//   P^T  = exp2(S^T*c - LSE)    dS^T = P^T o (dP^T - delta)        (registers -> bf16: P^T to TMEM, dS^T to shared memory)
//   dV  += P^T dO  (A operand read from TMEM)   dK += dS^T Q       (128 x 128 accumulators in TMEM; dK scaled at the end)
//   dQ^T = K^T dS^T         (128 x 64; staged through shared memory and added into dq_accum with bulk fp32
//                            reductions, cp.reduce.async.bulk, by four drain warps; scaled when converted to bf16)
// Pipeline: a loader warp keeps three (Q | dO) tiles and their LSE / delta rows in flight (the row statistics are
// fetched two tiles ahead so that their global-load latency is hidden); one thread issues every MMA, S^T / dP^T of
// tile i+1 ahead of the three accumulating GEMMs of tile i; sixteen softmax-gradient warps turn S^T / dP^T into
// P^T / dS^T (double buffered, so they never wait for the accumulating GEMMs); the drain warps empty dQ^T while the
// next tile's GEMMs run. CTAs are ordered heaviest key tile first. All MN-major operand forms (dO, Q, K^T, dS^T) are
// read from the very tiles TMA brought or the softmax warps wrote; no transposed copy exists. dK/dV need no atomics
// because the whole GQA group is reduced inside the CTA.
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
// Warp roles: 0 loader (TMA + per-row statistics), 1 MMA issue, 2..17 softmax-gradient warps (4 column groups of 16
// query columns x 4 TMEM lane quarters), 18..21 dQ drain warps (one per lane quarter).
constexpr int BWD_SM_WARPS = 16;
constexpr int BWD_DRAIN_WARPS = 4;
constexpr int BWD_THREADS = 32 * (2 + BWD_SM_WARPS + BWD_DRAIN_WARPS);  // 704

struct AttnBwdParams {
  CUtensorMap tmQ, tmK, tmV, tmdO;
  const float* lse;    // [B, Hq, Sq]
  const float* delta;  // [B, Hq, Sq]
  float* dq_accum;     // tiled fp32, see the drain warps
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  long long dk_row_stride, dv_row_stride, dk_batch_stride, dv_batch_stride;
  int* status;
  int B, Sq, Skv, Hq, Hk;
  int causal, window;
  float scale, scale_log2;
};

struct BwdCfg {
  static constexpr int STAGES = 3;                       // (Q | dO) tiles in flight: covers the TMA latency of ~1.5 us
  static constexpr int KV_BYTES = BWD_KV * BWD_D * 2;  // 32 KB
  static constexpr int Q_BYTES = BWD_Q * BWD_D * 2;    // 16 KB
  static constexpr int PT_BYTES = BWD_KV * BWD_Q * 2;  // 16 KB
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_Q = 2 * KV_BYTES;
  static constexpr int OFF_DST = OFF_Q + STAGES * 2 * Q_BYTES;  // dS^T, double buffered
  static constexpr int OFF_DQS = OFF_DST + 2 * PT_BYTES;        // dQ staging: 4 drain warps x [32 query rows][32 head-dim] fp32
  static constexpr int DQS_BYTES = 4 * 4096;
  static constexpr int OFF_STAT = OFF_DQS + DQS_BYTES;          // STAGES x {lse * log2e, delta} x 64 floats
  static constexpr int OFF_BAR = OFF_STAT + 2048;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // TMEM columns: S^T, dP^T, dQ^T (64 each), P^T as packed bf16 pairs (2 x 32), dV, dK (128 each)
  static constexpr uint32_t TM_S = 0, TM_DP = 64, TM_DQ = 128, TM_PT = 192, TM_DV = 256, TM_DK = 384;
};

__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using Cfg = BwdCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sQ = smem + Cfg::OFF_Q;
  uint8_t* sDST = smem + Cfg::OFF_DST;
  float* sStat = reinterpret_cast<float*>(smem + Cfg::OFF_STAT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // [3]
  uint64_t* qdo_empty = bars + 4;    // [3]
  uint64_t* stat_full = bars + 7;    // [3], 1 arrival each
  uint64_t* s_full = bars + 10;      // 1
  uint64_t* dp_full = bars + 11;     // 1
  uint64_t* pds_ready = bars + 12;   // 16 arrivals
  uint64_t* dq_full = bars + 13;     // 1
  uint64_t* dq_drained = bars + 14;  // 4 arrivals: the dQ^T accumulator has been read out of TMEM
  uint64_t* all_done = bars + 15;    // 1: every MMA of the CTA has executed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
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
    for (int i = 0; i < Cfg::STAGES; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
      mbar_init(&stat_full[i], 1);
    }
    mbar_init(all_done, 1);
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_ready, BWD_SM_WARPS);
    mbar_init(dq_full, 1);
    mbar_init(dq_drained, BWD_DRAIN_WARPS);
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
    // ------------------------------------------------------------ loader: TMA tiles + LSE / delta rows
    if (n_it > 0) {
      if (lane == 0) {
        mbar_expect_tx(kv_full, 2 * Cfg::KV_BYTES);
        tma5(sK, &p.tmK, kv_full, kv0, kv_head, b);
        tma5(sV, &p.tmV, kv_full, kv0, kv_head, b);
      }
      // LSE (scaled to log2) and delta of the 64 query rows of a tile: lane i holds rows i and i + 32. The loads run two
      // tiles ahead of their use so that their ~1 us latency never sits on the per-tile critical path.
      auto load_stats = [&](int it, float& l0, float& l1, float& d0, float& d1) {
        const int head = kv_head * G + it / n_qt;
        const int qrow0 = (qt_lo + it % n_qt) * BWD_Q;
        const long long so = ((long long)b * p.Hq + head) * p.Sq + qrow0;
        l0 = INFINITY; l1 = INFINITY; d0 = 0.f; d1 = 0.f;
        if (qrow0 + lane < p.Sq) { l0 = p.lse[so + lane] * 1.4426950408889634f; d0 = p.delta[so + lane]; }
        if (qrow0 + lane + 32 < p.Sq) { l1 = p.lse[so + lane + 32] * 1.4426950408889634f; d1 = p.delta[so + lane + 32]; }
      };
      float cl0, cl1, cd0, cd1, nl0 = INFINITY, nl1 = INFINITY, nd0 = 0.f, nd1 = 0.f;
      load_stats(0, cl0, cl1, cd0, cd1);
      if (n_it > 1) load_stats(1, nl0, nl1, nd0, nd1);
      for (int it = 0; it < n_it; ++it) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        const int head = kv_head * G + it / n_qt;
        const int qrow0 = (qt_lo + it % n_qt) * BWD_Q;
        if (!mbar_wait_warp(&qdo_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        if (lane == 0) {
          mbar_expect_tx(&qdo_full[s], 2 * Cfg::Q_BYTES);
          tma5(sQ + s * 2 * Cfg::Q_BYTES, &p.tmQ, &qdo_full[s], qrow0, head, b);
          tma5(sQ + s * 2 * Cfg::Q_BYTES + Cfg::Q_BYTES, &p.tmdO, &qdo_full[s], qrow0, head, b);
        }
        float* st = sStat + s * 128;
        st[lane] = cl0; st[lane + 32] = cl1; st[64 + lane] = cd0; st[64 + lane + 32] = cd1;
        __syncwarp();
        if (lane == 0) mbar_arrive(&stat_full[s]);
        cl0 = nl0; cl1 = nl1; cd0 = nd0; cd1 = nd1;
        if (it + 2 < n_it) load_stats(it + 2, nl0, nl1, nd0, nd1);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      constexpr uint32_t idesc_s = umma_idesc_f16(128, BWD_Q, 1, 0, 0);      // K Q^T, V dO^T
      constexpr uint32_t idesc_acc = umma_idesc_f16(128, BWD_D, 1, 0, 1);    // P^T dO, dS^T Q
      constexpr uint32_t idesc_dq = umma_idesc_f16(128, BWD_Q, 1, 1, 1);     // K^T dS^T
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDST0 = smem_u32(sDST);
      auto issue_sdp = [&](int it) {
        const uint32_t q = smem_u32(sQ + (it % Cfg::STAGES) * 2 * Cfg::Q_BYTES), dO = q + Cfg::Q_BYTES;
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
          if (!mbar_wait(&qdo_full[jn % Cfg::STAGES], (jn / Cfg::STAGES) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
        }
        tc_fence_after();
        // S^T / dP^T of the next tile go first: the softmax warps work on them while the three GEMMs below run
        if (it + 1 < n_it) issue_sdp(it + 1);
        const uint32_t q = smem_u32(sQ + (it % Cfg::STAGES) * 2 * Cfg::Q_BYTES), dO = q + Cfg::Q_BYTES;
        const uint32_t aDST = aDST0 + (it & 1) * Cfg::PT_BYTES;
        const uint32_t tPT = tmem_base + Cfg::TM_PT + (it & 1) * 32;
        // dV += P^T dO (P^T read from TMEM) ; dK += dS^T Q   (K = 64 query rows: 4 k-steps)
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem_base + Cfg::TM_DV, tPT + k * 8, umma_desc_sw128(dO + k * 2048, 8192, 1024), idesc_acc,
                      (it | k) ? 1u : 0u);
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
        umma_commit(&qdo_empty[it % Cfg::STAGES]);
        umma_commit(dq_full);
      }
      if (ok) umma_commit(all_done);
    }
  } else if (warp < 2 + BWD_SM_WARPS) {
    // ------------------------------------------------------------ softmax-gradient warps
    const int cg = (warp - 2) >> 2;     // column group: query columns [16*cg, 16*cg + 16) of the tile
    const int qd = warp & 3;            // TMEM lane quarter this warp may touch
    const int r = qd * 32 + lane;       // key row inside the tile == TMEM lane
    const int kv_idx = kv0 + r;
    const int c0 = cg * 16;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    bool ok = n_it > 0;
    for (int it = 0; it < n_it && ok; ++it) {
      const int qrow0 = (qt_lo + it % n_qt) * BWD_Q;
      const bool need_mask = (p.causal && kv0 + BWD_KV - 1 > qrow0 + offset) || (kv0 + BWD_KV > p.Skv) ||
                             (p.window > 0 && kv0 < qrow0 + BWD_Q - 1 + offset - p.window + 1);
      const int stg = it % Cfg::STAGES;
      if (!mbar_wait_warp(&stat_full[stg], (it / Cfg::STAGES) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      const float* st = sStat + stg * 128 + c0;
      float lse[16], dl[16];
#pragma unroll
      for (int i = 0; i < 16; i += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(st + i);
        const float4 d4 = *reinterpret_cast<const float4*>(st + 64 + i);
        lse[i] = a4.x; lse[i + 1] = a4.y; lse[i + 2] = a4.z; lse[i + 3] = a4.w;
        dl[i] = d4.x; dl[i + 1] = d4.y; dl[i + 2] = d4.z; dl[i + 3] = d4.w;
      }
      float pf[16];
      uint32_t pt[8], ds[8];
      if (!mbar_wait_warp(s_full, it & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v[16];
        tmem_ld16(tmem_base + Cfg::TM_S + lane_addr + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) pf[i] = exp2f(fmaf(__uint_as_float(v[i]), p.scale_log2, -lse[i]));
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int qi = qrow0 + c0 + i + offset;
            bool dead = kv_idx >= p.Skv;
            if (p.causal && kv_idx > qi) dead = true;
            if (p.window > 0 && kv_idx < qi - p.window + 1) dead = true;
            if (dead) pf[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; i += 2) pt[i / 2] = pack_bf16x2(pf[i], pf[i + 1]);
      }
      if (!mbar_wait_warp(dp_full, it & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t v[16];
        tmem_ld16(tmem_base + Cfg::TM_DP + lane_addr + c0, v);
        tmem_ld_wait();
        // dS without the softmax scale: dK and dQ are scaled once when they are written out
#pragma unroll
        for (int i = 0; i < 16; i += 2)
          ds[i / 2] = pack_bf16x2(pf[i] * (__uint_as_float(v[i]) - dl[i]), pf[i + 1] * (__uint_as_float(v[i + 1]) - dl[i + 1]));
      }
      // Buffer (it & 1) of P^T / dS^T was last read by the GEMMs of iteration it-2. Those were issued before the
      // S^T GEMM of this iteration and tcgen05 GEMMs of one thread execute in order, so s_full already covers them.
      {
        uint32_t* w = pt;
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(
                         tmem_base + Cfg::TM_PT + (it & 1) * 32 + lane_addr + cg * 8),
                     "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                     : "memory");
      }
      uint8_t* dstb = sDST + (it & 1) * Cfg::PT_BYTES;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int cc = cg * 2 + k;
        const int off = r * 128 + ((cc ^ (r & 7)) << 4);
        *reinterpret_cast<uint4*>(dstb + off) = make_uint4(ds[k * 4], ds[k * 4 + 1], ds[k * 4 + 2], ds[k * 4 + 3]);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
    }
    if (ok && n_it > 0) {
      if (mbar_wait_warp(all_done, 0, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) {
        tc_fence_after();
        // dK / dV accumulators -> bf16 rows: column groups 0,1 store the halves of dV, 2,3 the halves of dK (scaled)
        const bool row_ok = kv_idx < p.Skv;
        const bool is_dk = cg >= 2;
        const float mul = is_dk ? p.scale : 1.f;
        __nv_bfloat16* dst = (is_dk ? p.dK + (long long)b * p.dk_batch_stride + (long long)kv_idx * p.dk_row_stride
                                    : p.dV + (long long)b * p.dv_batch_stride + (long long)kv_idx * p.dv_row_stride) +
                             (long long)kv_head * BWD_D + (cg & 1) * 64;
        const uint32_t src = tmem_base + (is_dk ? Cfg::TM_DK : Cfg::TM_DV) + lane_addr + (cg & 1) * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld32(src + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[i]) * mul, __uint_as_float(v[i + 1]) * mul);
              o.y = pack_bf16x2(__uint_as_float(v[i + 2]) * mul, __uint_as_float(v[i + 3]) * mul);
              o.z = pack_bf16x2(__uint_as_float(v[i + 4]) * mul, __uint_as_float(v[i + 5]) * mul);
              o.w = pack_bf16x2(__uint_as_float(v[i + 6]) * mul, __uint_as_float(v[i + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + c * 32 + i) = o;
            }
          }
        }
      }
    } else if (n_it == 0 && cg == 0) {
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
  } else {
    // ------------------------------------------------------------ dQ drain warps
    // dQ^T tile in TMEM: lane = head-dim index, column = query row. Each warp owns one lane quarter and moves it in two
    // halves of 32 query rows: [32 query rows][32 head-dim] fp32 (4 KB, contiguous) staged in shared memory and added
    // into dq_accum with one bulk reduction each. dq_accum is tiled to match:
    // [b][head][q tile][lane quarter][64 query rows][32 head-dim].
    const int qd = warp & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    float* stage = reinterpret_cast<float*>(smem + Cfg::OFF_DQS) + qd * 1024;
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int head = kv_head * G + it / n_qt;
      const int qt = qt_lo + it % n_qt;
      float* dst = p.dq_accum + ((((long long)b * p.Hq + head) * n_qt_total + qt) * 4 + qd) * 2048;
      if (!mbar_wait_warp(dq_full, it & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld32(tmem_base + Cfg::TM_DQ + lane_addr, v0);
      tmem_ld32(tmem_base + Cfg::TM_DQ + lane_addr + 32, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the stage has been read
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; ++i) stage[i * 32 + lane] = __uint_as_float(h ? v1[i] : v0[i]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst + h * 1024),
                       "r"(smem_u32(stage)), "r"(4096)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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

// dq_accum (tiled as the backward kernel writes it) * scale -> bf16 dQ rows. One thread converts 4 values.
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dQ, int B, int Sq,
                                       int Hq, long long dq_row_stride, float scale) {
  const int n_qt = (Sq + BWD_Q - 1) / BWD_Q;
  const long long n = (long long)B * Hq * n_qt * (BWD_Q * BWD_D / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    // i enumerates float4 groups in storage order [tile][lane quarter (4)][query row (64)][head-dim (32)]
    const int di4 = i & 7;
    const int qi = (i >> 3) & 63;
    const int qd = (i >> 9) & 3;
    const long long t = i >> 11;           // (b * Hq + head) * n_qt + tile
    const int tile = t % n_qt;
    const long long bh = t / n_qt;
    const int head = bh % Hq;
    const long long bb = bh / Hq;
    const int srow = tile * BWD_Q + qi;
    if (srow >= Sq) continue;
    const float4 v = *reinterpret_cast<const float4*>(acc + i * 4);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale, v.y * scale), hi = __floats2bfloat162_rn(v.z * scale, v.w * scale);
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
                                                   a->dq_row_stride, a->scale);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
