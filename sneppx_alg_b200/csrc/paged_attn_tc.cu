// A3 on the tensor cores: paged decode attention for head size 128 with the query heads of one KV head as the
// N dimension of tcgen05 MMAs ("swap A/B": the 128 cached positions of a tile are the M rows).
//
// A work item is (sequence b, KV head hk, split); a CTA walks the 128-position tiles of its items in the block pool:
//   S^T = K_tile Q^T        M=128 positions, N=16 (query heads of this KV head, padded), K=D; fp32 in TMEM
//   P^T = exp2(S^T - m)     one cached position per thread (TMEM lane == position): G exponentials per thread
//                           instead of 128, the running max per head shared through shared memory
//   O^T += V_tile^T P^T     M=D (V consumed MN-major from its [position, d] tile), N=16, K=128 positions
// K and V tiles are gathered by TMA straight from the paged cache: one box per (cache block, 64-wide slab), placed so
// that the tile in shared memory has the same swizzled layout as a contiguous load. The cache is read once for all
// query heads of the KV head and there are no shuffles on the score path, which is what bounded the SIMT kernel
// (paged_attn.cu); here the kernel is bound by the TMA stream. Splits are merged by paged_merge_kernel.
// Serves the role of the reference's paged decode kernels (kernel/cuda/attention_cuda.cu:602-690).
#include "tc_common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int PT_BN = 128;      // cached positions per tile (M of the score MMA)
constexpr int PT_D = 128;       // head size
constexpr int PT_NQ = 16;       // N of both MMAs: query heads per KV head, padded
constexpr int PT_MAX_G = 8;
constexpr int PT_STAGES = 3;
constexpr int PT_THREADS = 192;  // warps 0-3: softmax / epilogue (TMEM lane quadrants 0-3), warp 4: MMA, warp 5: TMA
constexpr int PT_KV_BYTES = PT_BN * PT_D * 2;          // one K or V tile
constexpr int PT_Q_BYTES = PT_NQ * PT_D * 2;           // 4 KB: two buffers of Q rows, then the same size for P^T
constexpr int PT_OFF_P = 2 * PT_Q_BYTES;
constexpr int PT_OFF_ST = 3 * PT_Q_BYTES + 1024;       // stages: [K tile][V tile], 1024-byte aligned
constexpr int PT_OFF_BAR = PT_OFF_ST + PT_STAGES * 2 * PT_KV_BYTES;
constexpr int PT_SMEM = PT_OFF_BAR + 1024 + 1024;
constexpr int PT_TMEM_COLS = 32;                       // S^T at +0, O^T at +16

struct PagedTcParams {
  CUtensorMap tmQ, tmK, tmV;
  const int* block_table;
  const int* seq_lens;
  float* o_part;
  float* ml_part;
  int* status;
  int B, Hq, Hkv, block_size, max_blocks, nsplit;
  float scale_log2;
};

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

struct PtItem {
  int b, hk, split, len, t0, n_steps;
};

// Work item `item` of the (split, KV head, sequence) space, sequences fastest so that neighbouring CTAs hold different
// sequences; its tile range comes from the sequence length on the device.
__device__ __forceinline__ PtItem pt_item(const PagedTcParams& p, int item) {
  PtItem w;
  w.b = item % p.B;
  const int rest = item / p.B;
  w.hk = rest % p.Hkv;
  w.split = rest / p.Hkv;
  w.len = p.seq_lens[w.b];
  const int tiles = (w.len + PT_BN - 1) / PT_BN;
  const int per = (tiles + p.nsplit - 1) / p.nsplit;
  w.t0 = w.split * per;
  const int t1 = min(tiles, w.t0 + per);
  w.n_steps = t1 > w.t0 ? t1 - w.t0 : 0;
  return w;
}

// Persistent: one CTA per SM walks items blockIdx.x, blockIdx.x + gridDim.x, ...; the TMA warp runs ahead across item
// boundaries (the stage ring and every barrier phase are counted over the CTA's whole life), so the cache stream does
// not stop while an item's result is written out.
__global__ void __launch_bounds__(PT_THREADS, 1) paged_decode_tc_kernel(const __grid_constant__ PagedTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // two Q buffers
  uint8_t* sP = smem + PT_OFF_P;
  uint8_t* sSt = smem + PT_OFF_ST;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PT_OFF_BAR);
  uint64_t* q_full = bars;                 // [2]
  uint64_t* q_empty = bars + 2;            // [2]
  uint64_t* full = bars + 4;               // [PT_STAGES]
  uint64_t* empty = bars + 4 + PT_STAGES;  // [PT_STAGES]
  uint64_t* s_full = bars + 4 + 2 * PT_STAGES;
  uint64_t* p_full = s_full + 1;           // 4 arrivals (one per softmax warp)
  uint64_t* o_done = s_full + 2;
  uint64_t* red_bar = s_full + 3;          // 4 arrivals: per-warp maxima / sums are in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 4);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float (*s_red)[4][PT_MAX_G] = reinterpret_cast<float (*)[4][PT_MAX_G]>(smem + PT_OFF_BAR + 256);  // [2][4][G]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int n_items = p.B * p.Hkv * p.nsplit;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < PT_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
    mbar_init(red_bar, 4);
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmQ);
    tma_prefetch_desc(&p.tmK);
    tma_prefetch_desc(&p.tmV);
  }
  if (warp == 4) tmem_alloc(tmem_slot, PT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base, tO = tmem_base + 16;

  auto tma5 = [](void* dst, const CUtensorMap* m, uint64_t* bar, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(0), "r"(c1), "r"(c2),
        "r"(c3), "r"(c4)
        : "memory");
  };

  if (warp == 5) {
    // ------------------------------------------------------------ TMA producer (whole warp: one box per lane)
    const int bs = p.block_size;
    const int nchunk = PT_BN / bs;       // cache blocks per tile
    const int n_box = nchunk * 4;        // (K, V) x 2 slabs
    uint32_t gt = 0, qi = 0;             // tiles / non-empty items so far
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const PtItem w = pt_item(p, item);
      if (w.n_steps == 0) continue;
      const int qb = qi & 1;
      if (!mbar_wait_warp(&q_empty[qb], ((qi >> 1) & 1) ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) break;
      if (lane == 0) {
        mbar_expect_tx(&q_full[qb], PT_Q_BYTES);
        // 16 head rows from head hk*G on; rows past Hq are zero-filled
        tma5(sQ + qb * PT_Q_BYTES, &p.tmQ, &q_full[qb], w.hk * G, 0, 0, w.b);
      }
      ++qi;
      const int* tbl = p.block_table + (long long)w.b * p.max_blocks;
      for (int j = 0; j < w.n_steps; ++j, ++gt) {
        const int s = gt % PT_STAGES;
        const uint32_t ph = (gt / PT_STAGES) & 1;
        const int kv0 = (w.t0 + j) * PT_BN;
        if (!mbar_wait_warp(&empty[s], ph ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
        if (lane == 0) mbar_expect_tx(&full[s], 2 * PT_KV_BYTES);
        __syncwarp();
        uint8_t* st = sSt + s * 2 * PT_KV_BYTES;
        for (int t = lane; t < n_box; t += 32) {
          const int which = t / (nchunk * 2);   // 0: K, 1: V
          const int rem = t - which * nchunk * 2;
          const int i = rem >> 1, c = rem & 1;
          const int pos = kv0 + i * bs;
          // blocks past the end of the sequence are masked; any valid block keeps the tile finite
          const int blk = pos < w.len ? tbl[pos / bs] : tbl[0];
          tma5(st + which * PT_KV_BYTES + c * (PT_BN * 128) + i * bs * 128, which ? &p.tmV : &p.tmK, &full[s], 0, c,
               w.hk, blk);
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(PT_BN, PT_NQ, 1, 0, 0);   // A = K tile (K-major), B = Q (K-major)
      constexpr uint32_t idesc_pv = umma_idesc_f16(PT_D, PT_NQ, 1, 1, 0);    // A = V tile (MN-major), B = P^T (K-major)
      const uint32_t p0 = smem_u32(sP);
      uint32_t gt = 0, qi = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const PtItem w = pt_item(p, item);
        if (w.n_steps == 0) continue;
        const int qb = qi & 1;
        const uint32_t q0 = smem_u32(sQ + qb * PT_Q_BYTES);
        if (!mbar_wait(&q_full[qb], (qi >> 1) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        for (int j = 0; j < w.n_steps; ++j, ++gt) {
          const int s = gt % PT_STAGES;
          if (!mbar_wait(&full[s], (gt / PT_STAGES) & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t k0 = smem_u32(sSt + s * 2 * PT_KV_BYTES), v0 = k0 + PT_KV_BYTES;
#pragma unroll
          for (int c = 0; c < PT_D / 64; ++c)
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_ss(tS, umma_desc_sw128(k0 + c * (PT_BN * 128) + k * 32, 16, 1024),
                          umma_desc_sw128(q0 + c * (PT_NQ * 128) + k * 32, 16, 1024), idesc_qk, (c | k) ? 1u : 0u);
          umma_commit(s_full);
          if (!mbar_wait(p_full, gt & 1, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < PT_BN / 16; ++k)
            umma_f16_ss(tO, umma_desc_sw128(v0 + k * 2048, PT_BN * 128, 1024),
                        umma_desc_sw128(p0 + (k >> 2) * (PT_NQ * 128) + (k & 3) * 32, 16, 1024), idesc_pv,
                        (j | k) ? 1u : 0u);
          umma_commit(&empty[s]);
          if (j + 1 == w.n_steps) {
            umma_commit(o_done);
            umma_commit(&q_empty[qb]);
          }
        }
        ++qi;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue: thread t <-> position t / dim t
    const int t = threadIdx.x;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    // P^T rows of heads >= G stay zero for the whole kernel
    *reinterpret_cast<uint4*>(sP + t * 32) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(sP + t * 32 + 16) = make_uint4(0, 0, 0, 0);
    const uint32_t p_off = (t >> 6) * (PT_NQ * 128) + ((t & 7) << 1);   // slab and byte inside the 16-byte chunk
    const int p_chunk = (t & 63) >> 3;
    bool ok = true;
    uint32_t gt = 0, qi = 0, rc = 0;    // tiles, non-empty items, uses of red_bar so far
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const PtItem w = pt_item(p, item);
      const long long row0 = ((long long)w.b * p.Hq + (long long)w.hk * G) * p.nsplit + w.split;   // + g * nsplit
      if (w.n_steps == 0) {
        for (int g = 0; g < G; ++g) {
          const long long idx = row0 + (long long)g * p.nsplit;
          p.o_part[idx * PT_D + t] = 0.f;
          if (t == 0) { p.ml_part[idx * 2] = -INFINITY; p.ml_part[idx * 2 + 1] = 0.f; }
        }
        continue;
      }
      float m[PT_MAX_G], l[PT_MAX_G];
#pragma unroll
      for (int g = 0; g < PT_MAX_G; ++g) { m[g] = -INFINITY; l[g] = 0.f; }
      for (int j = 0; j < w.n_steps && ok; ++j, ++gt) {
        const int kv0 = (w.t0 + j) * PT_BN;
        const bool valid = kv0 + t < w.len;
        if (!mbar_wait_warp(s_full, gt & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        uint32_t r[16];
        tmem_ld16(tS + lane_addr, r);
        tmem_ld_wait();
        float sc[PT_MAX_G];
#pragma unroll
        for (int g = 0; g < PT_MAX_G; ++g) {
          sc[g] = (valid && g < G) ? __uint_as_float(r[g]) * p.scale_log2 : -INFINITY;
          float v = sc[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          if (lane == 0) s_red[rc & 1][warp][g] = v;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(red_bar);
        if (!mbar_wait_warp(red_bar, rc & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        float alpha[PT_MAX_G];
        bool rescale = false;
#pragma unroll
        for (int g = 0; g < PT_MAX_G; ++g) {
          const float mx = fmaxf(fmaxf(s_red[rc & 1][0][g], s_red[rc & 1][1][g]),
                                 fmaxf(s_red[rc & 1][2][g], s_red[rc & 1][3][g]));
          alpha[g] = 1.f;
          if ((mx > m[g] + 8.f || m[g] == -INFINITY) && mx != -INFINITY) {
            if (m[g] == -INFINITY) alpha[g] = 0.f;
            else { alpha[g] = exp2f(m[g] - mx); rescale = true; }
            m[g] = mx;
          }
        }
        ++rc;
#pragma unroll
        for (int g = 0; g < PT_MAX_G; ++g) {
          if (g < G) {
            const float pv = valid ? exp2f(sc[g] - m[g]) : 0.f;
            const __nv_bfloat16 pb = __float2bfloat16_rn(pv);
            // the row sum uses the rounded value so that l matches what the P V product sees
            l[g] = fmaf(l[g], alpha[g], __bfloat162float(pb));
            *reinterpret_cast<__nv_bfloat16*>(sP + p_off + g * 128 + ((p_chunk ^ (g & 7)) << 4)) = pb;
          }
        }
        // s_full of this tile completed after P V of the previous one (in-order tensor pipe): O^T and P^T are ours
        if (j > 0 && rescale) {
          uint32_t o[16];
          tmem_ld16(tO + lane_addr, o);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < PT_MAX_G; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
          tmem_st16(tO + lane_addr, o);
          tmem_st_wait();
        }
        if (kv0 + PT_BN > w.len) {
          // last tile of the sequence: rows past the end may hold anything (0 * NaN would poison O), clear their V rows
          const int s = gt % PT_STAGES;
          if (!mbar_wait_warp(&full[s], (gt / PT_STAGES) & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
          if (!valid) {
            uint8_t* vrow = sSt + s * 2 * PT_KV_BYTES + PT_KV_BYTES + t * 128;
#pragma unroll
            for (int c = 0; c < PT_D / 64; ++c)
#pragma unroll
              for (int i = 0; i < 8; ++i)
                *reinterpret_cast<uint4*>(vrow + c * (PT_BN * 128) + i * 16) = make_uint4(0, 0, 0, 0);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      if (!ok) break;
      // ---- partial result of this item for the merge kernel. Total row sums: every thread holds the partial sum of
      // its own positions.
#pragma unroll
      for (int g = 0; g < PT_MAX_G; ++g) {
        float v = l[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) s_red[rc & 1][warp][g] = v;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_bar);
      if (!mbar_wait_warp(red_bar, rc & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE) ||
          !mbar_wait_warp(o_done, qi & 1, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t o[16];
      tmem_ld16(tO + lane_addr, o);
      tmem_ld_wait();
      // the next item's first P V (which overwrites O^T) waits for this thread's next p_full arrival
      tc_fence_before();
#pragma unroll
      for (int g = 0; g < PT_MAX_G; ++g) {
        if (g < G) {
          const long long idx = row0 + (long long)g * p.nsplit;
          p.o_part[idx * PT_D + t] = __uint_as_float(o[g]);
          if (t == 0) {
            const int x = rc & 1;
            p.ml_part[idx * 2] = m[g] * 0.6931471805599453f;   // natural-log units for the merge
            p.ml_part[idx * 2 + 1] = s_red[x][0][g] + s_red[x][1][g] + s_red[x][2][g] + s_red[x][3][g];
          }
        }
      }
      ++rc;
      ++qi;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, PT_TMEM_COLS);
  }
}

void paged_merge_launch(const float* o_part, const float* ml_part, void* out, long long out_row_stride, int B, int Hq,
                        int D, int nsplit, cudaStream_t st);

}  // namespace sx
using namespace sx;

// Splits for the tensor-core kernel. It is persistent (one CTA per SM walks the (split, KV head, sequence) items), so
// splits only set the granularity: items of about six tiles keep the SMs evenly loaded, and there are at least two
// items per SM when the batch is small.
extern "C" int sx_paged_decode_tc_splits(int max_len, int ctas_per_split) {
  const int tiles = (max_len + PT_BN - 1) / PT_BN;
  const int by_size = (tiles + 5) / 6;
  const int by_fill = (2 * 148 + ctas_per_split - 1) / (ctas_per_split > 0 ? ctas_per_split : 1);
  int s = by_size > by_fill ? by_size : by_fill;
  if (s > tiles) s = tiles;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

// Same contract as sx_paged_decode (o_part: fp32 [B, Hq, nsplit, D], ml_part: fp32 [B, Hq, nsplit, 2] scratch);
// D = 128, block_size a divisor of 128 and a multiple of 8, at most 8 query heads per KV head.
extern "C" int sx_paged_decode_tc(const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                                  long long num_blocks, const int* block_table, const int* seq_lens, void* out,
                                  long long out_row_stride, float* o_part, float* ml_part, int B, int Hq, int Hkv, int D,
                                  int block_size, int max_blocks, int nsplit, float scale, int* status,
                                  cudaStream_t st) {
  if (D != PT_D || Hq % Hkv || Hq / Hkv > PT_MAX_G) return -1;
  if (block_size < 8 || PT_BN % block_size || (q_row_stride % 8)) return -2;
  PagedTcParams p;
  {
    // q [B, Hq, D]: dims {64, Hq, D/64, 1, B}; a box is 16 head rows x D as two swizzled 128-byte-row slabs
    uint64_t dims[5] = {64, (uint64_t)Hq, (uint64_t)(D / 64), 1, (uint64_t)B};
    uint64_t strides[4] = {(uint64_t)D * 2, 128, (uint64_t)q_row_stride * 2, (uint64_t)q_row_stride * 2};
    uint32_t box[5] = {64, PT_NQ, (uint32_t)(D / 64), 1, 1};
    int rc = make_tmap(&p.tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, q, dims, strides, box);
    if (rc) return rc;
  }
  {
    // cache [blocks, bs, Hkv, D]: dims {64, bs, D/64, Hkv, blocks}; a box is one block's rows of one 64-wide slab
    uint64_t dims[5] = {64, (uint64_t)block_size, (uint64_t)(D / 64), (uint64_t)Hkv, (uint64_t)num_blocks};
    uint64_t strides[4] = {(uint64_t)Hkv * D * 2, 128, (uint64_t)D * 2, (uint64_t)block_size * Hkv * D * 2};
    uint32_t box[5] = {64, (uint32_t)block_size, 1, 1, 1};
    int rc = make_tmap(&p.tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, k_cache, dims, strides, box);
    if (rc) return rc;
    rc = make_tmap(&p.tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, v_cache, dims, strides, box);
    if (rc) return rc;
  }
  p.block_table = block_table;
  p.seq_lens = seq_lens;
  p.o_part = o_part;
  p.ml_part = ml_part;
  p.status = status;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size; p.max_blocks = max_blocks; p.nsplit = nsplit;
  p.scale_log2 = scale * 1.4426950408889634f;
  static bool set = false;
  if (!set) {
    if (cudaFuncSetAttribute(paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PT_SMEM) !=
        cudaSuccess)
      return -10;
    set = true;
  }
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  }
  const long long items = (long long)B * Hkv * nsplit;
  paged_decode_tc_kernel<<<(unsigned)(items < sms ? items : sms), PT_THREADS, PT_SMEM, st>>>(p);
  paged_merge_launch(o_part, ml_part, out, out_row_stride, B, Hq, D, nsplit, st);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
