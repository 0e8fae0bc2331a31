// A3: paged decode attention (one query token per sequence, KV in a block pool addressed through block tables,
//     split along the sequence with a log-sum-exp merge) and
// A4: KV append fused with RoPE (rotates the new Q and K rows, scatters K/V into the block pool by slot mapping).
// Cache layout [num_blocks, block_size, Hkv, D] bf16, block tables [B, max_blocks] int32 - the layout of the
// reference's paged kernels (kernel/cuda/attention_cuda.cu:602-690, 839-865), whose decode kernel re-reads K/V once
// per query head; here one CTA serves all query heads of a KV head so the cache is streamed once.
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr int PA_TILE = 128;   // positions per tile == threads per CTA
constexpr int PA_MAX_G = 8;    // query heads per KV head

template <int D>
__global__ void __launch_bounds__(PA_TILE) paged_decode_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_row_stride, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, const int* __restrict__ seq_lens,
    float* __restrict__ o_part, float* __restrict__ ml_part, int Hq, int Hkv, int block_size, int max_blocks,
    int nsplit, float scale) {
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ float s_q[PA_MAX_G][D];
  __shared__ float s_p[PA_MAX_G][PA_TILE];
  __shared__ long long s_row[PA_TILE];
  __shared__ float s_red[PA_MAX_G][4];
  __shared__ float s_alpha[PA_MAX_G];
  const int len = seq_lens[b];
  const int per = (len + nsplit - 1) / nsplit;
  const int p0 = split * per, p1 = min(len, p0 + per);
  for (int i = tid; i < G * D; i += PA_TILE) {
    const int g = i / D, d = i % D;
    s_q[g][d] = __bfloat162float(q[(long long)b * q_row_stride + (long long)(hk * G + g) * D + d]) * scale;
  }
  float m_run[PA_MAX_G], l_run[PA_MAX_G], acc[PA_MAX_G];
#pragma unroll
  for (int g = 0; g < PA_MAX_G; ++g) { m_run[g] = -INFINITY; l_run[g] = 0.f; acc[g] = 0.f; }
  __syncthreads();
  for (int t0 = p0; t0 < p1; t0 += PA_TILE) {
    const int pos = t0 + tid;
    const bool valid = pos < p1;
    long long rowoff = 0;
    if (valid) {
      const int blk = block_table[(long long)b * max_blocks + pos / block_size];
      rowoff = (((long long)blk * block_size + pos % block_size) * Hkv + hk) * D;
    }
    s_row[tid] = valid ? rowoff : -1;
    // scores of this thread's position against all G query heads
    float sc[PA_MAX_G];
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) sc[g] = 0.f;
    if (valid) {
      const __nv_bfloat16* kr = k_cache + rowoff;
      for (int d = 0; d < D; d += 8) {
        float kv[8];
        unpack8(ld8(kr + d), kv);
#pragma unroll
        for (int g = 0; g < PA_MAX_G; ++g)
          if (g < G) {
#pragma unroll
            for (int j = 0; j < 8; ++j) sc[g] += kv[j] * s_q[g][d + j];
          }
      }
    }
    // tile max per head
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) {
      if (g < G) {
        const float v = warp_max(valid ? sc[g] : -INFINITY);
        if (lane == 0) s_red[g][warp] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) {
      if (g < G) {
        const float tm = fmaxf(fmaxf(s_red[g][0], s_red[g][1]), fmaxf(s_red[g][2], s_red[g][3]));
        const float mn = fmaxf(m_run[g], tm);
        const float pr = valid ? __expf(sc[g] - mn) : 0.f;
        s_p[g][tid] = pr;
        const float alpha = (m_run[g] == -INFINITY) ? 0.f : __expf(m_run[g] - mn);
        if (tid == 0) s_alpha[g] = alpha;
        m_run[g] = mn;
        sc[g] = pr;
      }
    }
    __syncthreads();
    // row sums
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) {
      if (g < G) {
        const float v = warp_sum(sc[g]);
        if (lane == 0) s_red[g][warp] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g)
      if (g < G) l_run[g] = l_run[g] * s_alpha[g] + (s_red[g][0] + s_red[g][1] + s_red[g][2] + s_red[g][3]);
    // P V: thread = head-dim index
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < PA_MAX_G; ++g)
        if (g < G) acc[g] *= s_alpha[g];
      const int n = min(PA_TILE, p1 - t0);
      for (int t = 0; t < n; ++t) {
        const float v = __bfloat162float(v_cache[s_row[t] + tid]);
#pragma unroll
        for (int g = 0; g < PA_MAX_G; ++g)
          if (g < G) acc[g] += s_p[g][t] * v;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int g = 0; g < PA_MAX_G; ++g) {
    if (g < G) {
      const long long idx = ((long long)b * Hq + hk * G + g) * nsplit + split;
      if (tid < D) o_part[idx * D + tid] = acc[g];
      if (tid == 0) {
        ml_part[idx * 2] = m_run[g];
        ml_part[idx * 2 + 1] = l_run[g];
      }
    }
  }
}

__global__ void paged_merge_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                   __nv_bfloat16* __restrict__ out, long long out_row_stride, int Hq, int D, int nsplit) {
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

}  // namespace sx
using namespace sx;

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
  if (D == 128)
    paged_decode_kernel<128><<<grid, PA_TILE, 0, st>>>((const __nv_bfloat16*)q, q_row_stride,
                                                       (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                                       block_table, seq_lens, o_part, ml_part, Hq, Hkv, block_size,
                                                       max_blocks, nsplit, scale);
  else
    paged_decode_kernel<64><<<grid, PA_TILE, 0, st>>>((const __nv_bfloat16*)q, q_row_stride,
                                                      (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
                                                      block_table, seq_lens, o_part, ml_part, Hq, Hkv, block_size,
                                                      max_blocks, nsplit, scale);
  paged_merge_kernel<<<dim3(B, Hq), D, 0, st>>>(o_part, ml_part, (__nv_bfloat16*)out, out_row_stride, Hq, D, nsplit);
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
