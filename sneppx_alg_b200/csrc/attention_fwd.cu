// A1: flash attention forward on tcgen05 (sm_100a).
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles X in {A, B}, each served
// by its own softmax warpgroup, and walks the visible 128-row KV tiles:
//   S_X = Q_X K^T       tcgen05.mma SS, fp32 in TMEM
//   P_X = exp2(S_X - m) one query row per thread (TMEM lane == row, no shuffles); P is written back
//                       as packed bf16 over the S columns it came from
//   O_X += P_X V        tcgen05.mma TS: P straight from TMEM, V consumed MN-major from its [kv, d] tile
// The MMA warp ping-pongs the two tiles (PV(A,j), QK(A,j+1), PV(B,j), QK(B,j+1), ...), so the tensor
// pipe works on one tile while the other tile's warpgroup does its softmax. tcgen05.mma executes in
// issue order, which is what makes the S/P aliasing safe. The running max is only refreshed when
// it grew by more than 2^8, so rescaling O in TMEM is rare. Causal / sliding-window masks, GQA head
// mapping and the differential-attention V mapping (two score heads share one V head) are index
// arithmetic; nothing is materialised. An optional block mask (one byte per 128 x 128 score tile, per head or
// shared) removes whole tiles from the walk: a step whose tile is masked for both query tiles is neither loaded nor
// multiplied (block-sparse / flex-attention patterns at tile granularity).
// Takes the place of the reference's SIMT flash-attention forward, GQA and block-sparse kernels
// (kernel/cuda/attention_cuda.cu:37-328, 498-573, 1154-1230) and its empty "v3" kernel (:1262-1286).
#include <limits.h>
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int ATT_BM = 128;   // rows per q tile (two per CTA)
constexpr int ATT_BN = 128;
constexpr int ATT_THREADS = 320;  // TMA warp, MMA warp, 2 x 4 softmax warps

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
  const uint8_t* block_mask;   // optional [B or 1][Hq or 1][q tiles][kv tiles], non-zero = tile takes part
  long long bm_batch_stride, bm_head_stride;
  int bm_kv_tiles;
};

template <int D>
struct AttnCfg {
  static constexpr int Q_BYTES = ATT_BM * D * 2;   // one q tile
  static constexpr int KV_BYTES = ATT_BN * D * 2;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;  // per tile: S/P at +0 (128 cols), O at +128; tile B at +256
};

// Visible KV tile range [lo, hi) of a 128-row q tile starting at q0.
__device__ __forceinline__ void kv_range(const AttnFwdParams& p, int q0, int& lo, int& hi) {
  const int offset = p.Skv - p.Sq;
  lo = 0;
  hi = (p.Skv + ATT_BN - 1) / ATT_BN;
  if (q0 >= p.Sq) { hi = 0; return; }
  if (p.causal) {
    const int last = q0 + ATT_BM - 1 + offset;
    hi = last < 0 ? 0 : min(hi, last / ATT_BN + 1);
  }
  if (p.window > 0) {
    const int first = q0 + offset - p.window + 1;
    if (first > 0) lo = first / ATT_BN;
  }
  if (hi < lo) hi = lo;
}

template <int D, bool MASK>
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using Cfg = AttnCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + Cfg::OFF_K;
  uint8_t* sV = smem + Cfg::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [2 tiles]
  uint64_t* p_full = bars + 11;       // [2 tiles]
  uint64_t* o_done = bars + 13;       // [2 tiles]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: better tail behaviour under the causal mask
  const int pair = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hk);
  const int v_head = kv_head / p.v_head_div;
  const int q0 = pair * 2 * ATT_BM;

  int lo[2], hi[2];
  kv_range(p, q0, lo[0], hi[0]);
  kv_range(p, q0 + ATT_BM, lo[1], hi[1]);
  // union range walked by the loaders; tile X takes part in step j when lo[X] <= j < hi[X]
  int jlo = INT_MAX, jhi = 0;
#pragma unroll
  for (int x = 0; x < 2; ++x)
    if (hi[x] > lo[x]) { jlo = min(jlo, lo[x]); jhi = max(jhi, hi[x]); }
  // tile X takes part in the step of kv tile jt?
  const uint8_t* bm = MASK ? p.block_mask + b * p.bm_batch_stride + head * p.bm_head_stride : nullptr;
  auto on = [&](int x, int jt) -> bool {
    if (jt < lo[x] || jt >= hi[x]) return false;
    if constexpr (!MASK) return true;
    else return bm[(long long)(pair * 2 + x) * p.bm_kv_tiles + jt] != 0;
  };
  // next kv tile after jt that any of the two tiles takes part in (-1: none)
  auto next_step = [&](int jt) -> int {
    if constexpr (!MASK) {
      return jt + 1 < jhi ? jt + 1 : -1;   // without a mask every tile of the union range is taken
    } else {
      for (++jt; jt < jhi; ++jt)
        if (on(0, jt) || on(1, jt)) return jt;
      return -1;
    }
  };
  const int first_step = jhi > jlo ? next_step(jlo - 1) : -1;
  const int n_steps = first_step >= 0 ? 1 : 0;   // only "are there any" is used below

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
    }
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

  auto tma5 = [](void* dst, const CUtensorMap* m, uint64_t* bar, int c1, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(0), "r"(c1), "r"(0),
        "r"(c3), "r"(c4)
        : "memory");
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_steps > 0) {
      mbar_expect_tx(q_full, 2 * Cfg::Q_BYTES);
      tma5(sQ, &p.tmQ, q_full, q0, head, b);
      tma5(sQ + Cfg::Q_BYTES, &p.tmQ, q_full, q0 + ATT_BM, head, b);
      int j = 0;   // steps taken so far
      for (int jt = first_step; jt >= 0; jt = next_step(jt), ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int kv0 = jt * ATT_BN;
        if (!mbar_wait(&k_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&k_full[s], Cfg::KV_BYTES);
        tma5(sK + s * Cfg::KV_BYTES, &p.tmK, &k_full[s], kv0, kv_head, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(&v_full[s], Cfg::KV_BYTES);
        tma5(sV + s * Cfg::KV_BYTES, &p.tmV, &v_full[s], kv0, v_head, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(ATT_BM, ATT_BN, 1, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(ATT_BM, D, 1, 0, 1);
      auto issue_qk = [&](int x, int j) {
        const uint32_t a0 = smem_u32(sQ + x * Cfg::Q_BYTES), b0 = smem_u32(sK + (j & 1) * Cfg::KV_BYTES);
        const uint32_t d = tmem_base + x * 256;
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ss(d, umma_desc_sw128(a0 + c * (ATT_BM * 128) + k * 32, 16, 1024),
                        umma_desc_sw128(b0 + c * (ATT_BN * 128) + k * 32, 16, 1024), idesc_qk, (c | k) ? 1u : 0u);
        umma_commit(&s_full[x]);
      };
      // steps each tile takes part in: total, and so far (gives barrier parities and accumulate flags)
      int total[2] = {0, 0}, cnt[2] = {0, 0};
      for (int jt = first_step; jt >= 0; jt = next_step(jt))
        for (int x = 0; x < 2; ++x) total[x] += on(x, jt) ? 1 : 0;
      bool ok = mbar_wait(q_full, 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = mbar_wait(&k_full[0], 0, s_abort, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        for (int x = 0; x < 2; ++x)
          if (on(x, first_step)) issue_qk(x, 0);
        umma_commit(&k_empty[0]);
      }
      int j = 0;   // steps taken so far; K / V ring slot and phase follow it
      for (int jt = first_step; jt >= 0 && ok; ++j) {
        const int nxt = next_step(jt);
        const bool more = nxt >= 0;
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        if (more && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) {
          ok = false;
          break;
        }
        for (int x = 0; x < 2 && ok; ++x) {
          if (on(x, jt)) {
            if (!mbar_wait(&p_full[x], cnt[x] & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
            const uint32_t b0 = smem_u32(sV + (j & 1) * Cfg::KV_BYTES);
            const uint32_t dO = tmem_base + x * 256 + 128, aP = tmem_base + x * 256;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_f16_ts(dO, aP + k * 8, umma_desc_sw128(b0 + k * 2048, ATT_BN * 128, 1024), idesc_pv,
                          (cnt[x] | k) ? 1u : 0u);
            ++cnt[x];
            if (cnt[x] == total[x]) umma_commit(&o_done[x]);  // last step of this tile
          }
          if (more && on(x, nxt)) issue_qk(x, j + 1);
        }
        umma_commit(&v_empty[j & 1]);
        if (more) umma_commit(&k_empty[(j + 1) & 1]);
        jt = nxt;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    const int x = (warp - 2) >> 2;          // which q tile
    const int qd = warp & 3;                // TMEM lane quadrant of this warp
    const int row = qd * 32 + lane;         // row inside the tile == TMEM lane
    const int q_idx = q0 + x * ATT_BM + row;
    const int offset = p.Skv - p.Sq;
    const uint32_t lane_addr = static_cast<uint32_t>(qd * 32) << 16;
    const uint32_t tS = tmem_base + x * 256 + lane_addr;
    const uint32_t tO = tS + 128;
    int n_mine = 0;   // steps this tile takes part in
    for (int jt = lo[x]; jt < hi[x]; ++jt) n_mine += on(x, jt) ? 1 : 0;
    float m_used = -INFINITY;  // running (possibly stale) max, log2 domain
    float l = 0.f;
    bool ok = true;
    int hi_k = p.Skv - 1;  // last visible key index for this row
    if (p.causal) hi_k = min(hi_k, q_idx + offset);
    const int lo_k = p.window > 0 ? q_idx + offset - p.window + 1 : INT_MIN;
    for (int jt = lo[x], j = 0; jt < hi[x] && ok; ++jt) {
      if (!on(x, jt)) continue;
      const int kv0 = jt * ATT_BN;
      if (!mbar_wait_warp(&s_full[x], j & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int qt0 = q0 + x * ATT_BM;
      const bool need_mask = (p.causal && kv0 + ATT_BN - 1 > qt0 + offset) || (kv0 + ATT_BN > p.Skv) ||
                             (p.window > 0 && kv0 < qt0 + ATT_BM - 1 + offset - p.window + 1);
      uint32_t r[ATT_BN];
#pragma unroll
      for (int c = 0; c < ATT_BN / 32; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_ld_wait();
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < ATT_BN; ++i) {
          const int kv = kv0 + i;
          if (kv > hi_k || kv < lo_k) r[i] = 0xff800000u;  // -inf
          mx = fmaxf(mx, __uint_as_float(r[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < ATT_BN; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      mx *= p.scale_log2;
      float alpha = 1.f;
      bool rescale = false;
      if ((mx > m_used + 8.f || m_used == -INFINITY) && mx != -INFINITY) {
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - mx);
        rescale = (m_used != -INFINITY);
        m_used = mx;
      }
      l *= alpha;
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      float lsum = 0.f;
#pragma unroll
      for (int i = 0; i < ATT_BN; i += 2) {
        const float v0 = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, -m_sub));
        const float v1 = exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -m_sub));
        const uint32_t pb = pack_bf16x2(v0, v1);
        r[i / 2] = pb;
        // row sum from the rounded values so that l matches what P V sees
        lsum += __uint_as_float(pb << 16) + __uint_as_float(pb & 0xffff0000u);
      }
      l += lsum;
      // s_full(j) was committed after P V of step j-1 (in-order pipe), so O and the S/P columns are ours
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + c * 32, o);
        }
      }
      tmem_st32(tS, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_st32(tS + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
      ++j;
    }
    if (ok && n_mine > 0) {
      if (mbar_wait_warp(&o_done[x], 0, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) {
        tc_fence_after();
        const float inv_l = l > 0.f ? 1.f / l : 0.f;
        const bool row_ok = q_idx < p.Sq;
        __nv_bfloat16* orow = p.O + ((long long)b * p.Sq + q_idx) * p.o_row_stride + (long long)head * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 w;
              w.x = pack_bf16x2(__uint_as_float(o[i]) * inv_l, __uint_as_float(o[i + 1]) * inv_l);
              w.y = pack_bf16x2(__uint_as_float(o[i + 2]) * inv_l, __uint_as_float(o[i + 3]) * inv_l);
              w.z = pack_bf16x2(__uint_as_float(o[i + 4]) * inv_l, __uint_as_float(o[i + 5]) * inv_l);
              w.w = pack_bf16x2(__uint_as_float(o[i + 6]) * inv_l, __uint_as_float(o[i + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
            }
          }
        }
        if (row_ok && p.lse)
          p.lse[((long long)b * p.Hq + head) * p.Sq + q_idx] =
              (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    } else if (n_mine <= 0) {
      // no visible keys for this tile: zero output
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
  p.block_mask = (const uint8_t*)a->block_mask;
  p.bm_batch_stride = a->bm_batch_stride;
  p.bm_head_stride = a->bm_head_stride;
  p.bm_kv_tiles = (a->Skv + ATT_BN - 1) / ATT_BN;
  dim3 grid((a->Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), a->Hq, a->B);
  if (a->D == 128) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_fwd_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<128>::SMEM_BYTES) != cudaSuccess ||
          cudaFuncSetAttribute(attn_fwd_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<128>::SMEM_BYTES) != cudaSuccess) return -10;
      set = true;
    }
    if (p.block_mask) attn_fwd_kernel<128, true><<<grid, ATT_THREADS, AttnCfg<128>::SMEM_BYTES, st>>>(p);
    else attn_fwd_kernel<128, false><<<grid, ATT_THREADS, AttnCfg<128>::SMEM_BYTES, st>>>(p);
  } else {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(attn_fwd_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<64>::SMEM_BYTES) != cudaSuccess ||
          cudaFuncSetAttribute(attn_fwd_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               AttnCfg<64>::SMEM_BYTES) != cudaSuccess) return -10;
      set = true;
    }
    if (p.block_mask) attn_fwd_kernel<64, true><<<grid, ATT_THREADS, AttnCfg<64>::SMEM_BYTES, st>>>(p);
    else attn_fwd_kernel<64, false><<<grid, ATT_THREADS, AttnCfg<64>::SMEM_BYTES, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
