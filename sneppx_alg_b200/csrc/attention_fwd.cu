// A1: flash attention forward on tcgen05 (sm_100a).
//
// One CTA owns 128 query rows of one (batch, head). Per 128-row KV tile:
//   S = Q K^T        tcgen05.mma SS, fp32 in TMEM (two S buffers so QK^T of tile j+1 overlaps softmax j)
//   P = exp2(S - m)  four softmax warps, one query row per thread (TMEM lane == row, no shuffles);
//                    P is written as bf16 into a 128B-swizzled smem tile
//   O += P V         tcgen05.mma SS with V consumed MN-major straight from its [kv, d] layout
// The running max is only refreshed when it grew by more than 2^8 (the stale max keeps every
// exponent bounded), which makes the O rescale in TMEM rare. Causal / sliding-window masks, GQA
// head mapping and the differential-attention V mapping (two score heads share one V head) are
// index arithmetic in the kernel; nothing is materialised.
// Takes the place of the reference's SIMT flash-attention forward, GQA and block-sparse kernels
// (kernel/cuda/attention_cuda.cu:37-328, 498-573, 1154-1230) and its empty "v3" kernel (:1262-1286).
#include <limits.h>
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int ATT_BM = 128;
constexpr int ATT_BN = 128;
constexpr int ATT_THREADS = 192;
constexpr int KV_STAGES = 2;

struct AttnFwdParams {
  CUtensorMap tmQ, tmK, tmV;
  __nv_bfloat16* O;   // [B, Sq, Hq, D]
  float* lse;         // [B, Hq, Sq]  (natural log)
  int* status;
  long long o_row_stride;  // elements between consecutive tokens of O
  int B, Sq, Skv, Hq, Hk;
  int v_head_div;  // V head = (K head) / v_head_div
  int causal, window;  // window <= 0: unlimited
  float scale_log2;    // softmax scale * log2(e)
};

template <int D>
struct AttnCfg {
  static constexpr int Q_BYTES = ATT_BM * D * 2;
  static constexpr int KV_BYTES = ATT_BN * D * 2;
  static constexpr int P_BYTES = ATT_BM * ATT_BN * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;  // S0 | S1 | O (128 + 128 + D columns used)
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using Cfg = AttnCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint8_t* sP = smem + Cfg::OFF_P;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2]
  uint64_t* s_empty = bars + 11;      // [2]
  uint64_t* p_full = bars + 13;       // 1
  uint64_t* o_done = bars + 14;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: better tail behaviour under the causal mask
  const int q_tile = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hk);
  const int v_head = kv_head / p.v_head_div;
  const int q0 = q_tile * ATT_BM;
  const int offset = p.Skv - p.Sq;  // query i sees keys <= i + offset under the causal mask

  int tile_lo = 0;
  int tile_hi = (p.Skv + ATT_BN - 1) / ATT_BN;  // exclusive
  if (p.causal) {
    const int last = q0 + ATT_BM - 1 + offset;
    tile_hi = min(tile_hi, last / ATT_BN + 1);
    if (last < 0) tile_hi = 0;
  }
  if (p.window > 0) {
    const int first = q0 + offset - p.window + 1;
    if (first > 0) tile_lo = first / ATT_BN;
  }
  const int n_tiles = max(tile_hi - tile_lo, 0);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmQ);
    tma_prefetch_desc(&p.tmK);
    tma_prefetch_desc(&p.tmV);
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S0 = tmem_base;           // S buffers at columns 0 and 128
  const uint32_t tmem_O = tmem_base + 256;

  auto tma5 = [](void* dst, const CUtensorMap* m, uint64_t* bar, int c1, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(0), "r"(c1), "r"(0),
        "r"(c3), "r"(c4)
        : "memory");
  };

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
      tma5(sQ, &p.tmQ, q_full, q0, head, b);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv0 = (tile_lo + j) * ATT_BN;
        if (!mbar_wait(&k_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&k_full[s], Cfg::KV_BYTES);
        tma5(sK + s * Cfg::KV_BYTES, &p.tmK, &k_full[s], kv0, kv_head, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&v_full[s], Cfg::KV_BYTES);
        tma5(sV + s * Cfg::KV_BYTES, &p.tmV, &v_full[s], kv0, v_head, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(ATT_BM, ATT_BN, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(ATT_BM, D, 1, 0, 1);
      auto issue_qk = [&](int j) {
        const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + (j & 1) * Cfg::KV_BYTES);
        const uint32_t d = tmem_S0 + (j & 1) * ATT_BN;
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(d, umma_desc_sw128(a0 + c * (ATT_BM * 128) + k * 32, 16, 1024),
                        umma_desc_sw128(b0 + c * (ATT_BN * 128) + k * 32, 16, 1024), idesc_qk, (c | k) ? 1u : 0u);
        umma_commit(&k_empty[j & 1]);
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = mbar_wait(&k_full[0], 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          const int jn = j + 1;
          if (!mbar_wait(&k_full[jn & 1], (jn >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          if (!mbar_wait(&s_empty[jn & 1], ((jn >> 1) & 1) ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          issue_qk(jn);
        }
        if (!mbar_wait(p_full, j & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a0 = smem_u32(sP), b0 = smem_u32(sV + (j & 1) * Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(tmem_O, umma_desc_sw128(a0 + c * (ATT_BM * 128) + k * 32, 16, 1024),
                        umma_desc_sw128(b0 + (c * 4 + k) * 2048, ATT_BN * 128, 1024), idesc_pv,
                        (j | c | k) ? 1u : 0u);
        umma_commit(&v_empty[j & 1]);
        umma_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax / correction / epilogue
    const int qd = warp & 3;
    const int row = qd * 32 + lane;           // row inside the tile == TMEM lane
    const int q_idx = q0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    float m_used = -INFINITY;  // running (possibly stale) max, log2 domain
    float l = 0.f;
    bool ok = n_tiles > 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int kv0 = (tile_lo + j) * ATT_BN;
      if (!mbar_wait_warp(&s_full[j & 1], (j >> 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_S0 + (j & 1) * ATT_BN + lane_addr;
      const bool need_mask = (p.causal && kv0 + ATT_BN - 1 > q0 + offset) || (kv0 + ATT_BN > p.Skv) ||
                             (p.window > 0 && kv0 < q0 + ATT_BM - 1 + offset - p.window + 1);
      int hi = p.Skv - 1;  // last visible key index for this row
      if (p.causal) hi = min(hi, q_idx + offset);
      const int lo = p.window > 0 ? q_idx + offset - p.window + 1 : INT_MIN;
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < ATT_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv > hi || kv < lo) v = -INFINITY;
          }
          mx = fmaxf(mx, v);
        }
      }
      mx *= p.scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_used + 8.f || m_used == -INFINITY) {
        if (mx != -INFINITY) {
          alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
          rescale = (m_used != -INFINITY);
          m_used = mx;
        }
      }
      l *= alpha;
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      // pass 2: probabilities, packed to bf16 in registers
      uint32_t pk[ATT_BN / 2];
#pragma unroll
      for (int c = 0; c < ATT_BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float v0 = exp2f(__uint_as_float(r[i]) * p.scale_log2 - m_sub);
          float v1 = exp2f(__uint_as_float(r[i + 1]) * p.scale_log2 - m_sub);
          if (need_mask) {
            const int kv = kv0 + c * 32 + i;
            if (kv > hi || kv < lo) v0 = 0.f;
            if (kv + 1 > hi || kv + 1 < lo) v1 = 0.f;
          }
          const uint32_t pb = pack_bf16x2(v0, v1);
          pk[c * 16 + i / 2] = pb;
          // accumulate the row sum from the rounded values so that l matches what P V sees
          const __nv_bfloat162 pv = *reinterpret_cast<const __nv_bfloat162*>(&pb);
          l += __low2float(pv) + __high2float(pv);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[j & 1]);
      // P buffer and O are free once P V of the previous tile has completed
      if (j > 0) {
        if (!mbar_wait_warp(o_done, (j - 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem_O + lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tmem_O + lane_addr + c * 32, r);
          }
          tmem_st_wait();
        }
      }
      // write P (row-major [128 x 128] bf16) as two 128B-swizzled K-major tiles
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const int tile = ch >> 3, cc = ch & 7;
        uint4 val = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(sP + tile * (ATT_BM * 128) + row * 128 + ((cc ^ (row & 7)) << 4)) = val;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && n_tiles > 0) {
      if (mbar_wait_warp(o_done, (n_tiles - 1) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) {
        tc_fence_after();
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = q_idx < p.Sq;
        __nv_bfloat16* orow = p.O + ((long long)b * p.Sq + q_idx) * p.o_row_stride + (long long)head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem_O + lane_addr + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[i]) * inv_l, __uint_as_float(r[i + 1]) * inv_l);
              o.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
              o.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l);
              o.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = o;
            }
          }
        }
        if (row_ok && p.lse)
          p.lse[((long long)b * p.Hq + head) * p.Sq + q_idx] =
              (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    } else if (n_tiles == 0) {
      // no visible keys: zero output
      if (q_idx < p.Sq) {
        __nv_bfloat16* orow = p.O + ((long long)b * p.Sq + q_idx) * p.o_row_stride + (long long)head * D;
        for (int i = 0; i < D; i += 8) *reinterpret_cast<uint4*>(orow + i) = make_uint4(0, 0, 0, 0);
        if (p.lse) p.lse[((long long)b * p.Hq + head) * p.Sq + q_idx] = -INFINITY;
      }
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

// 5-D map over a [B, S, H, D] view (token stride `row_stride` elements): dims
// {64, S, D/64, H, B}; one box brings a [128 tokens x D] tile as D/64 swizzled 128-byte-row slabs.
static int make_attn_map(CUtensorMap* tm, const void* base, int B, int S, int H, int D, long long row_stride,
                         long long batch_stride, int box_rows) {
  uint64_t dims[5] = {64, (uint64_t)S, (uint64_t)(D / 64), (uint64_t)H, (uint64_t)B};
  uint64_t strides[4] = {(uint64_t)row_stride * 2, 128, (uint64_t)D * 2, (uint64_t)batch_stride * 2};
  uint32_t box[5] = {64, (uint32_t)box_rows, (uint32_t)(D / 64), 1, 1};
  return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, box);
}

}  // namespace sx
using namespace sx;

extern "C" int sx_attn_fwd(const SxAttnArgs* a, cudaStream_t st) {
  if (a->D != 64 && a->D != 128) return -1;
  if (a->Hq % a->Hk) return -2;
  if ((a->q_row_stride % 8) || (a->k_row_stride % 8) || (a->v_row_stride % 8) || (a->o_row_stride % 8)) return -3;
  AttnFwdParams p;
  const int v_heads = a->Hk / (a->v_head_div > 0 ? a->v_head_div : 1);
  int rc = make_attn_map(&p.tmQ, a->Q, a->B, a->Sq, a->Hq, a->D, a->q_row_stride, a->q_batch_stride, ATT_BM);
  if (rc) return rc;
  rc = make_attn_map(&p.tmK, a->K, a->B, a->Skv, a->Hk, a->D, a->k_row_stride, a->k_batch_stride, ATT_BN);
  if (rc) return rc;
  rc = make_attn_map(&p.tmV, a->V, a->B, a->Skv, v_heads, a->D, a->v_row_stride, a->v_batch_stride, ATT_BN);
  if (rc) return rc;
  p.O = (__nv_bfloat16*)a->O;
  p.lse = a->lse;
  p.status = a->status;
  p.o_row_stride = a->o_row_stride;
  p.B = a->B; p.Sq = a->Sq; p.Skv = a->Skv; p.Hq = a->Hq; p.Hk = a->Hk;
  p.v_head_div = a->v_head_div > 0 ? a->v_head_div : 1;
  p.causal = a->causal; p.window = a->window;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  dim3 grid((a->Sq + ATT_BM - 1) / ATT_BM, a->Hq, a->B);
  if (a->D == 128) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<128>::SMEM_BYTES) != cudaSuccess) return -10;
      set = true;
    }
    attn_fwd_kernel<128><<<grid, ATT_THREADS, AttnCfg<128>::SMEM_BYTES, st>>>(p);
  } else {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<64>::SMEM_BYTES) != cudaSuccess) return -10;
      set = true;
    }
    attn_fwd_kernel<64><<<grid, ATT_THREADS, AttnCfg<64>::SMEM_BYTES, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
