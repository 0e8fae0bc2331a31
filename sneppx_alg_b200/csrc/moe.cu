// M1: SER router (softmax over experts -> top-k -> renormalise, lowest index wins ties), routing metadata built
//     on the device (per-expert counts, 128-row padded offsets, token permutation, tile -> expert table), and the
//     local halves of F5/F6: row gather into the expert-sorted buffer and the top-k weighted combine, forward and
//     backward. The expert-parallel versions of gather/combine live in comm_moe.cu and write/read peer memory.
// Router math follows the reference (algorithms/ser/core/route.c:94-157: softmax over all experts, top-k,
// renormalise; loss.c:31-69 load-balance loss E * sum_e f_e p_e; route.c:251 z-loss = mean(logit^2)); its CUDA
// gating kernel handled E <= 64 with one warp per token and a top-1-only dispatch (algorithms/ser/cuda/ser_cuda.cu:23-162).
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr int ROUTER_MAX_E = 256;
constexpr int ROUTER_MAX_K = 8;

// One warp per token. logits [T, E] fp32. Outputs: probs [T, E] (optional), topk_idx [T, k], topk_w [T, k],
// counts[E] (+1 per selection), psum_partial [gridDim, E] sum of probs per expert, zsum_partial [gridDim] sum logit^2.
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, float* __restrict__ probs,
                                                          int* __restrict__ topk_idx, float* __restrict__ topk_w,
                                                          int* __restrict__ counts, float* __restrict__ psum_partial,
                                                          float* __restrict__ zsum_partial, int T, int E, int k,
                                                          int renorm) {
  __shared__ float s_psum[ROUTER_MAX_E];
  __shared__ float s_z[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_psum[e] = 0.f;
  __syncthreads();
  float zacc = 0.f;
  constexpr int PER = ROUTER_MAX_E / 32;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? logits[(long long)t * E + e] : -INFINITY;
      if (e < E) zacc += v[i] * v[i];
      mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;
      sum += v[i];
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      v[i] *= inv;
      const int e = lane + 32 * i;
      if (e < E) {
        if (probs) probs[(long long)t * E + e] = v[i];
        atomicAdd(&s_psum[e], v[i]);
      }
    }
    // k rounds of arg-max; ties resolved to the lowest expert index
    float wsel[ROUTER_MAX_K];
    int isel[ROUTER_MAX_K];
    float wsum = 0.f;
    for (int r = 0; r < k; ++r) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        if (e < E && (v[i] > best)) { best = v[i]; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      wsel[r] = best;
      isel[r] = bi;
      wsum += best;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (lane + 32 * i == bi) v[i] = -1.f;  // remove from further rounds
    }
    if (lane == 0) {
      const float rn = renorm ? 1.f / wsum : 1.f;
      for (int r = 0; r < k; ++r) {
        topk_idx[(long long)t * k + r] = isel[r];
        topk_w[(long long)t * k + r] = wsel[r] * rn;
        if (counts) atomicAdd(&counts[isel[r]], 1);
      }
    }
  }
  zacc = warp_sum(zacc);
  if (lane == 0) s_z[warp] = zacc;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) psum_partial[(long long)blockIdx.x * E + e] = s_psum[e];
  if (threadIdx.x == 0) {
    float z = 0.f;
    for (int i = 0; i < 8; ++i) z += s_z[i];
    zsum_partial[blockIdx.x] = z;
  }
}

// Single CTA: padded exclusive offsets (each expert segment rounded up to 128 rows), tile -> expert table,
// per-expert [begin, end) padded row ranges for the grouped wgrad, and cursors reset for the slot assignment.
// meta layout (int32): [0..E) offsets, [E] total padded rows, then cursors [E].
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursors,
                                   int* __restrict__ tile_group, int* __restrict__ k_ranges, int E, int max_tiles) {
  __shared__ int s_off[ROUTER_MAX_E + 1];
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = o;
      o += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) {
      cursors[e] = 0;
      if (k_ranges) {
        k_ranges[2 * e] = s_off[e];
        k_ranges[2 * e + 1] = s_off[e + 1];
      }
    }
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= row) lo = mid; else hi = mid - 1;
      }
      g = lo;
    }
    tile_group[t] = g;
  }
}

// slot[t, r] = offsets[e] + (arrival order within e); row_token[slot] = t (pad rows keep -1).
__global__ void moe_assign_slots_kernel(const int* __restrict__ topk_idx, const int* __restrict__ offsets,
                                        int* __restrict__ cursors, int* __restrict__ slot, int* __restrict__ row_token,
                                        long long TK, int k) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < TK;
       i += (long long)gridDim.x * blockDim.x) {
    const int e = topk_idx[i];
    const int s = offsets[e] + atomicAdd(&cursors[e], 1);
    slot[i] = s;
    row_token[s] = (int)(i / k);
  }
}

// xs[row] = x[row_token[row]] (zeros for pad rows). One warp per row, 16-byte vectors.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                  const int* __restrict__ total_rows, __nv_bfloat16* __restrict__ xs, int d,
                                  int max_rows) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  const int rows = min(*total_rows, max_rows);
  for (int r = warp; r < rows; r += nw) {
    const int t = row_token[r];
    for (int c = lane * 8; c < d; c += 256) {
      bf16x8 v;
      if (t >= 0) v = ld8(x + (long long)t * d + c);
      else *reinterpret_cast<uint4*>(&v) = make_uint4(0, 0, 0, 0);
      st8(xs + (long long)r * d + c, v);
    }
  }
}

// y[t] = sum_r w[t, r] * ys[slot[t, r]]  (+ base[t] when given, e.g. shared-expert output)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ slot,
                                   const float* __restrict__ w, const __nv_bfloat16* __restrict__ base,
                                   __nv_bfloat16* __restrict__ y, int T, int d, int k) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nw) {
    for (int c = lane * 8; c < d; c += 256) {
      float acc[8];
      if (base) unpack8(ld8(base + (long long)t * d + c), acc);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      }
      for (int r = 0; r < k; ++r) {
        const int s = slot[(long long)t * k + r];
        if (s < 0) continue;  // dropped by the capacity limit
        const float ww = w[(long long)t * k + r];
        float v[8];
        unpack8(ld8(ys + (long long)s * d + c), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += ww * v[j];
      }
      st8(y + (long long)t * d + c, pack8(acc));
    }
  }
}

// Backward of combine: dys[slot[t, r]] = w[t, r] * dy[t] ; dw[t, r] = <dy[t], ys[slot[t, r]]>. Pad rows of dys are
// zero-filled by the caller (memset) so the grouped GEMMs see zeros there.
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ys,
                                       const int* __restrict__ slot, const float* __restrict__ w,
                                       __nv_bfloat16* __restrict__ dys, float* __restrict__ dw, int T, int d, int k) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nw) {
    for (int r = 0; r < k; ++r) {
      const int s = slot[(long long)t * k + r];
      if (s < 0) {
        if (lane == 0) dw[(long long)t * k + r] = 0.f;
        continue;
      }
      const float ww = w[(long long)t * k + r];
      float dot = 0.f;
      for (int c = lane * 8; c < d; c += 256) {
        float g[8], v[8], o[8];
        unpack8(ld8(dy + (long long)t * d + c), g);
        unpack8(ld8(ys + (long long)s * d + c), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          dot += g[j] * v[j];
          o[j] = ww * g[j];
        }
        st8(dys + (long long)s * d + c, pack8(o));
      }
      dot = warp_sum(dot);
      if (lane == 0) dw[(long long)t * k + r] = dot;
    }
  }
}

// Backward of gather: dx[t] = sum_r dxs[slot[t, r]]
__global__ void moe_gather_bwd_kernel(const __nv_bfloat16* __restrict__ dxs, const int* __restrict__ slot,
                                      __nv_bfloat16* __restrict__ dx, int T, int d, int k) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T; t += nw) {
    for (int c = lane * 8; c < d; c += 256) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < k; ++r) {
        const int s = slot[(long long)t * k + r];
        if (s < 0) continue;
        float v[8];
        unpack8(ld8(dxs + (long long)s * d + c), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[j];
      }
      st8(dx + (long long)t * d + c, pack8(acc));
    }
  }
}

}  // namespace sx
using namespace sx;

extern "C" int sx_router_parts(void) { return 148 * 6; }  // CTAs (and partial-sum rows): enough warps in flight to hide the per-token latency chain

// counts must be zeroed by the caller. psum_partial: [sx_router_parts() * E], zsum_partial: [sx_router_parts()].
extern "C" int sx_router_topk(const float* logits, float* probs, int* topk_idx, float* topk_w, int* counts,
                              float* psum_partial, float* zsum_partial, int T, int E, int k, int renorm,
                              cudaStream_t st) {
  if (E > ROUTER_MAX_E || k > ROUTER_MAX_K || k < 1 || k > E) return -1;
  router_topk_kernel<<<sx_router_parts(), 256, 0, st>>>(logits, probs, topk_idx, topk_w, counts, psum_partial,
                                                        zsum_partial, T, E, k, renorm);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// offsets: int32 [E+1]; cursors: int32 [E]; tile_group: int32 [max_tiles]; k_ranges: int32 [2E] (optional);
// slot: int32 [T*k]; row_token: int32 [max_tiles*128], filled with -1 here.
extern "C" int sx_moe_plan(const int* counts, const int* topk_idx, int* offsets, int* cursors, int* tile_group,
                           int* k_ranges, int* slot, int* row_token, int T, int E, int k, int max_tiles,
                           cudaStream_t st) {
  if (E > ROUTER_MAX_E) return -1;
  cudaMemsetAsync(row_token, 0xff, sizeof(int) * (size_t)max_tiles * 128, st);
  moe_offsets_kernel<<<1, 256, 0, st>>>(counts, offsets, cursors, tile_group, k_ranges, E, max_tiles);
  const long long TK = (long long)T * k;
  const int blocks = (int)((TK + 255) / 256 < 1184 ? (TK + 255) / 256 : 1184);
  moe_assign_slots_kernel<<<blocks < 1 ? 1 : blocks, 256, 0, st>>>(topk_idx, offsets, cursors, slot, row_token, TK, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_moe_gather(const void* x, const int* row_token, const int* total_rows, void* xs, int d, int max_rows,
                             cudaStream_t st) {
  if (d % 8) return -1;
  moe_gather_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)x, row_token, total_rows, (__nv_bfloat16*)xs, d,
                                             max_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_moe_combine(const void* ys, const int* slot, const float* w, const void* base, void* y, int T, int d,
                              int k, cudaStream_t st) {
  if (d % 8) return -1;
  moe_combine_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)ys, slot, w, (const __nv_bfloat16*)base,
                                              (__nv_bfloat16*)y, T, d, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_moe_combine_bwd(const void* dy, const void* ys, const int* slot, const float* w, void* dys, float* dw,
                                  int T, int d, int k, cudaStream_t st) {
  if (d % 8) return -1;
  moe_combine_bwd_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)ys, slot, w,
                                                  (__nv_bfloat16*)dys, dw, T, d, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_moe_gather_bwd(const void* dxs, const int* slot, void* dx, int T, int d, int k, cudaStream_t st) {
  if (d % 8) return -1;
  moe_gather_bwd_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)dxs, slot, (__nv_bfloat16*)dx, T, d, k);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
