// A3: paged decode attention (one query token per sequence, KV in a block pool addressed through block tables,
//     split along the sequence with a log-sum-exp merge) and
// A4: KV append fused with RoPE (rotates the new Q and K rows, scatters K/V into the block pool by slot mapping).
// Cache layout [num_blocks, block_size, Hkv, D] bf16, block tables [B, max_blocks] int32 - the layout of the
// reference's paged kernels (kernel/cuda/attention_cuda.cu:602-690, 839-865), whose decode kernel re-reads K/V once
// per query head; here one CTA serves all query heads of a KV head so the cache is streamed once.
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr int PA_TILE = 128;   // threads per CTA
constexpr int PA_MAX_G = 8;    // query heads per KV head
constexpr int PA_NST = 8;      // cp.async ring depth per lane
constexpr int PA_TBL = 1024;   // block-table entries staged per CTA

// One CTA: (sequence b, KV head hk, split). A K/V row (D bf16) is read by D/8 adjacent lanes with one 16-byte load
// each, so a warp reads 2 (D=128) or 4 (D=64) whole rows per load instruction, fully coalesced; the lanes of a row
// keep their 8-wide slice of every query head in registers, reduce the partial dot products with shuffles and
// accumulate P*V for their slice. Every lane group runs its own online softmax over the positions it owns; groups
// are merged through shared memory at the end, splits by paged_merge_kernel.
template <int D, int GT>
__global__ void __launch_bounds__(PA_TILE) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_row_stride, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, const int* __restrict__ seq_lens,
    float* __restrict__ o_part, float* __restrict__ ml_part, int Hq, int Hkv, int block_size, int max_blocks,
    int nsplit, float scale) {
  constexpr int LPR = D / 8;            // lanes per row
  constexpr int RPW = 32 / LPR;         // rows per warp-wide load
  constexpr int NGRP = (PA_TILE / 32) * RPW;
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int sub = lane % LPR, grp = warp * RPW + lane / LPR;
  // one shared buffer: the cp.async ring while streaming, the per-group partial results for the final merge
  constexpr int RING_BYTES = PA_NST * 2 * PA_TILE * 16;
  constexpr int MERGE_BYTES = NGRP * GT * (D + 2) * 4;
  __shared__ __align__(16) uint8_t s_raw[RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES];
  uint4 (*s_ring)[2][PA_TILE] = reinterpret_cast<uint4 (*)[2][PA_TILE]>(s_raw);
  float (*s_acc)[GT][D] = reinterpret_cast<float (*)[GT][D]>(s_raw);
  float (*s_m)[GT] = reinterpret_cast<float (*)[GT]>(s_raw + NGRP * GT * D * 4);
  float (*s_l)[GT] = reinterpret_cast<float (*)[GT]>(s_raw + NGRP * GT * D * 4 + NGRP * GT * 4);
  const int len = seq_lens[b];
  const int per = (len + nsplit - 1) / nsplit;
  const int p0 = split * per, p1 = min(len, p0 + per);
  float qr[GT][8], m[GT], l[GT], acc[GT][8];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (g < G) {
      unpack8(ld8(q + (long long)b * q_row_stride + (long long)(hk * G + g) * D + sub * 8), qr[g]);
#pragma unroll
      for (int j = 0; j < 8; ++j) qr[g][j] *= scale;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) qr[g][j] = 0.f;
    }
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[g][j] = 0.f;
  }
  // Block-table entries of this CTA's position range, staged once (a lookup on the load path costs a shared-memory
  // read instead of a dependent global load).
  __shared__ int s_tbl[PA_TBL];
  const int* tbl = block_table + (long long)b * max_blocks;
  const int blk0 = p0 / block_size;
  const int nblk = p1 > p0 ? (p1 - 1) / block_size - blk0 + 1 : 0;
  const bool tbl_staged = nblk <= PA_TBL;
  if (tbl_staged)
    for (int i = tid; i < nblk; i += PA_TILE) s_tbl[i] = tbl[blk0 + i];
  __syncthreads();
  // Per-lane ring of 16-byte K and V pieces filled by cp.async: PA_NST - 1 rows per lane group are in flight while one
  // is consumed, without holding registers for them. A lane reads back exactly the bytes it copied, so the only
  // synchronisation is its own cp.async.wait_group.
  const int n_it = p1 > p0 ? (p1 - p0 + NGRP - 1) / NGRP : 0;   // uniform for the whole CTA
  auto issue = [&](int i) {
    const int pos = p0 + i * NGRP + grp;
    if (i < n_it && pos < p1) {
      const int blk = tbl_staged ? s_tbl[pos / block_size - blk0] : tbl[pos / block_size];
      const long long row = (((long long)blk * block_size + pos % block_size) * Hkv + hk) * D + sub * 8;
      const uint32_t dk = (uint32_t)__cvta_generic_to_shared(&s_ring[i % PA_NST][0][tid]);
      const uint32_t dv = (uint32_t)__cvta_generic_to_shared(&s_ring[i % PA_NST][1][tid]);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk), "l"(k_cache + row) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dv), "l"(v_cache + row) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < PA_NST - 1; ++i) issue(i);
  for (int i = 0; i < n_it; ++i) {
    issue(i + PA_NST - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(PA_NST - 1) : "memory");
    const int pos = p0 + i * NGRP + grp;
    const bool valid = pos < p1;
    float kv[8], vv[8];
    if (valid) {
      const uint4 kq = s_ring[i % PA_NST][0][tid], vq = s_ring[i % PA_NST][1][tid];
      unpack8(*reinterpret_cast<const bf16x8*>(&kq), kv);
      unpack8(*reinterpret_cast<const bf16x8*>(&vq), vv);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) { kv[j] = 0.f; vv[j] = 0.f; }
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float sc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) sc = fmaf(kv[j], qr[g][j], sc);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
      if (valid) {
        if (sc > m[g]) {
          const float alpha = __expf(m[g] - sc);   // exp(-inf) = 0 on the first row
          l[g] *= alpha;
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[g][j] *= alpha;
          m[g] = sc;
        }
        const float pr = __expf(sc - m[g]);
        l[g] += pr;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[g][j] = fmaf(pr, vv[j], acc[g][j]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();   // the ring is dead from here on: its storage holds the merge buffers
  // merge the lane groups
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    if (sub == 0) { s_m[grp][g] = m[g]; s_l[grp][g] = l[g]; }
#pragma unroll
    for (int j = 0; j < 8; ++j) s_acc[grp][g][sub * 8 + j] = acc[g][j];
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += PA_TILE) {
    const int g = i / D, d = i % D;
    float mm = -INFINITY;
#pragma unroll
    for (int r = 0; r < NGRP; ++r) mm = fmaxf(mm, s_m[r][g]);
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int r = 0; r < NGRP; ++r) {
      const float w = (s_m[r][g] == -INFINITY) ? 0.f : __expf(s_m[r][g] - mm);
      ll += s_l[r][g] * w;
      oo += s_acc[r][g][d] * w;
    }
    const long long idx = ((long long)b * Hq + hk * G + g) * nsplit + split;
    o_part[idx * D + d] = oo;
    if (d == 0) {
      ml_part[idx * 2] = mm;
      ml_part[idx * 2 + 1] = ll;
    }
  }
}

__global__ void paged_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                   __nv_bfloat16* __restrict__ out, long long out_row_stride, int Hq, int D, int nsplit) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may start its prologue
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)b * Hq + h) * nsplit;
  float m = -INFINITY;
  for (int s = 0; s < nsplit; ++s) m = fmaxf(m, ml_part[(base + s) * 2]);
  float l = 0.f, o = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const float ms = ml_part[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
    l += ml_part[(base + s) * 2 + 1] * w;
    if (d < D) o += o_part[(base + s) * D + d] * w;
  }
  if (d < D) out[(long long)b * out_row_stride + (long long)h * D + d] = __float2bfloat16(l > 0.f ? o / l : 0.f);
}

// One warp per (token, head). Heads [0, Hq) are queries (rotated in place), [Hq, Hq+Hkv) keys (rotated, written to the
// cache), [Hq+Hkv, Hq+2Hkv) values (copied to the cache). qkv row = token, row stride in elements.
__global__ void kv_append_kernel(__nv_bfloat16* __restrict__ qkv, long long row_stride, const float* __restrict__ cos_t,
                                 const float* __restrict__ sin_t, const int* __restrict__ pos,
                                 const int* __restrict__ slot, __nv_bfloat16* __restrict__ k_cache,
                                 __nv_bfloat16* __restrict__ v_cache, int T, int Hq, int Hkv, int D, int rotate) {
  const int heads = Hq + 2 * Hkv;
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)T * heads) return;
  const int h = w % heads;
  const int t = w / heads;
  __nv_bfloat16* row = qkv + (long long)t * row_stride + (long long)h * D;
  const int half = D >> 1;
  const int p = pos[t];
  const int sl = slot[t];
  if (h < Hq + Hkv) {
    __nv_bfloat16* dst = (h >= Hq && sl >= 0) ? k_cache + ((long long)sl * Hkv + (h - Hq)) * D : nullptr;
    for (int i = lane; i < half; i += 32) {
      float a = __bfloat162float(row[i]), b2 = __bfloat162float(row[i + half]);
      if (rotate) {
        const float c = cos_t[(long long)p * half + i], s = sin_t[(long long)p * half + i];
        const float ra = a * c - b2 * s, rb = b2 * c + a * s;
        a = ra;
        b2 = rb;
        row[i] = __float2bfloat16(a);
        row[i + half] = __float2bfloat16(b2);
      }
      if (dst) {
        dst[i] = __float2bfloat16(a);
        dst[i + half] = __float2bfloat16(b2);
      }
    }
  } else if (sl >= 0) {
    __nv_bfloat16* dst = v_cache + ((long long)sl * Hkv + (h - Hq - Hkv)) * D;
    for (int i = lane; i < D; i += 32) dst[i] = row[i];
  }
}

// Shared with the tensor-core decode kernel (paged_attn_tc.cu).
void paged_merge_launch(const float* o_part, const float* ml_part, void* out, long long out_row_stride, int B, int Hq,
                        int D, int nsplit, cudaStream_t st) {
  paged_merge_kernel<<<dim3(B, Hq), D, 0, st>>>(o_part, ml_part, (__nv_bfloat16*)out, out_row_stride, Hq, D, nsplit);
}

}  // namespace sx
using namespace sx;

// Splits along the sequence: enough CTAs to fill the machine a few times over, at least 256 positions per split.
extern "C" int sx_paged_decode_splits2(int max_len, int ctas_per_split) {
  int by_len = (max_len + 255) / 256;
  int want = (148 * 4 + ctas_per_split - 1) / (ctas_per_split > 0 ? ctas_per_split : 1);
  int s = by_len < want ? by_len : want;
  return s < 1 ? 1 : (s > 64 ? 64 : s);
}
extern "C" int sx_paged_decode_splits(int max_len) {
  int s = (max_len + 1023) / 1024;
  return s < 1 ? 1 : (s > 32 ? 32 : s);
}

// o_part: fp32 [B, Hq, nsplit, D]; ml_part: fp32 [B, Hq, nsplit, 2] scratch.
extern "C" int sx_paged_decode(const void* q, long long q_row_stride, const void* k_cache, const void* v_cache,
                               const int* block_table, const int* seq_lens, void* out, long long out_row_stride,
                               float* o_part, float* ml_part, int B, int Hq, int Hkv, int D, int block_size,
                               int max_blocks, int nsplit, float scale, cudaStream_t st) {
  if (Hq % Hkv || Hq / Hkv > PA_MAX_G || (D != 64 && D != 128)) return -1;
  dim3 grid(B, Hkv, nsplit);
  const int G = Hq / Hkv;
#define SX_PD(DD, GG)                                                                                              \
  paged_decode_kernel<DD, GG><<<grid, PA_TILE, 0, st>>>((const __nv_bfloat16*)q, q_row_stride,                       \
                                                        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, \
                                                        block_table, seq_lens, o_part, ml_part, Hq, Hkv, block_size, \
                                                        max_blocks, nsplit, scale)
  if (D == 128) {
    if (G == 1) SX_PD(128, 1); else if (G == 2) SX_PD(128, 2); else if (G <= 4) SX_PD(128, 4); else SX_PD(128, 8);
  } else {
    if (G == 1) SX_PD(64, 1); else if (G == 2) SX_PD(64, 2); else if (G <= 4) SX_PD(64, 4); else SX_PD(64, 8);
  }
#undef SX_PD
  paged_merge_launch(o_part, ml_part, out, out_row_stride, B, Hq, D, nsplit, st);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_kv_append(void* qkv, long long row_stride, const float* cos_t, const float* sin_t, const int* pos,
                            const int* slot, void* k_cache, void* v_cache, int T, int Hq, int Hkv, int D, int rotate,
                            cudaStream_t st) {
  const long long warps = (long long)T * (Hq + 2 * Hkv);
  if (warps == 0) return 0;
  const int blocks = (int)((warps * 32 + 255) / 256);
  kv_append_kernel<<<blocks, 256, 0, st>>>((__nv_bfloat16*)qkv, row_stride, cos_t, sin_t, pos, slot,
                                           (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, T, Hq, Hkv, D, rotate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
