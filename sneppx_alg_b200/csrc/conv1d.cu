// C1: causal depthwise conv1d (kernel width <= 4) with optional SiLU, channels-last [B, L, C] bf16,
// forward and backward, halo aware: an optional [B, K-1, C] "previous tokens" tensor supplies the left
// context (chunked prefill, decode and context-parallel ranks pass the tail of the previous chunk) and
// the final K-1 tokens can be written out as the next state.
// The reference's conv kernels limit L to one thread block (algorithms/hss/cuda/hss_cuda_extended.cu:208-226)
// and its Mamba-2 block copies instead of convolving (kernel/arch/mamba2.c:82-84).
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr int CONV_MAXK = 4;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float silu_grad(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

// One thread: 8 channels x CONV_TL consecutive positions. The 8 x K weights and the bias live in registers and the
// K-1 previous inputs slide through registers, so each input vector is loaded once and each output costs one 16-byte
// load and one 16-byte store; consecutive threads own consecutive channel vectors (coalesced rows).
constexpr int CONV_TL = 16;
template <int K>
__global__ void __launch_bounds__(256) conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ prev,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ bias,
                                                         __nv_bfloat16* __restrict__ y,
                                                         __nv_bfloat16* __restrict__ state_out, int B, int L, int C,
                                                         int act, long long xld) {
  const int cv = C >> 3;
  const int lchunks = (L + CONV_TL - 1) / CONV_TL;
  const long long total = (long long)B * lchunks * cv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % cv) * 8;
    const long long bl = idx / cv;
    const int l0 = (int)(bl % lchunks) * CONV_TL;
    const int b = (int)(bl / lchunks);
    float wv[CONV_MAXK][8], bv[8];
#pragma unroll
    for (int k = 0; k < CONV_MAXK; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[k][j] = (k < K) ? __bfloat162float(w[(c + j) * K + k]) : 0.f;
    if (bias) unpack8(ld8(bias + c), bv);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) bv[j] = 0.f;
    }
    // hist[i] = input at position l - (K-1) + i for the current l; hist[K-1] is the current input
    float hist[CONV_MAXK][8];
#pragma unroll
    for (int i = 0; i < CONV_MAXK; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) hist[i][j] = 0.f;
    for (int i = 0; i < K - 1; ++i) {
      const int ls = l0 - (K - 1) + i;
      if (ls >= 0) unpack8(ld8(x + ((long long)b * L + ls) * xld + c), hist[i]);
      else if (prev) unpack8(ld8(prev + ((long long)b * (K - 1) + (K - 1 + ls)) * C + c), hist[i]);
    }
    const int l1 = min(L, l0 + CONV_TL);
    for (int lb = l0; lb < l1; lb += 4) {
      bf16x8 raw4[4];   // four independent 16-byte loads in flight per thread
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (lb + u < l1) raw4[u] = ld8(x + ((long long)b * L + lb + u) * xld + c);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int l = lb + u;
        if (l >= l1) break;
        const bf16x8 raw = raw4[u];
        unpack8(raw, hist[K - 1]);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = bv[j];
#pragma unroll
        for (int k = 0; k < CONV_MAXK; ++k)
          if (k < K) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(hist[k][j], wv[k][j], acc[j]);
          }
        if (act) {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = silu_f(acc[j]);
        }
        st8(y + ((long long)b * L + l) * C + c, pack8(acc));
        if (state_out && l >= L - (K - 1)) st8(state_out + ((long long)b * (K - 1) + (l - (L - (K - 1)))) * C + c, raw);
#pragma unroll
        for (int i = 0; i < CONV_MAXK - 1; ++i)
          if (i < K - 1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) hist[i][j] = hist[i + 1][j];
          }
      }
    }
  }
}

// dx and per-CTA partials of dw / dbias. A CTA is 32 channel groups of 4 (one per lane: 256 contiguous bytes per
// row) by 8 runs of CONV_BTL consecutive positions (one per warp). A thread walks its run once: the last K inputs and
// the last K pre-activation gradients slide through registers, so every x and dy value is loaded once (plus the K-1
// row overlap between runs) and dx is stored once. Four channels per thread keep the kernel near 100 registers (two
// CTAs per SM); with eight it needed 205 and ran at one. The 8 warps add their dw / db into shared memory and the CTA
// writes one partial row; conv1d_reduce_partials sums the rows.
constexpr int CONV_BTL = 16;
constexpr int CONV_BV = 4;
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&f)[CONV_BV]) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&f)[CONV_BV]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&a);
  r.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}
template <int K>
__global__ void __launch_bounds__(256, 2) conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ prev,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ bias,
                                                            __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                                            int B, int L, int C, int act, long long xld) {
  constexpr int V = CONV_BV;
  __shared__ float s_acc[32][(CONV_MAXK + 1) * V + 1];
  const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
  const int cv = C / V;
  const int v = blockIdx.x * 32 + lane;
  const bool live = v < cv;
  const int c = v * V;
  for (int i = threadIdx.x; i < 32 * ((CONV_MAXK + 1) * V + 1); i += 256) (&s_acc[0][0])[i] = 0.f;
  __syncthreads();
  if (live) {
    float wv[K][V], bv[V], dwacc[K][V], dbacc[V];
    if (K == 4) {   // a channel's four taps are 8 contiguous bytes
#pragma unroll
      for (int j = 0; j < V; ++j) {
        float t[4];
        ld4(w + (c + j) * 4, t);
#pragma unroll
        for (int k = 0; k < K; ++k) wv[k][j] = t[k];
      }
    } else {
#pragma unroll
      for (int k = 0; k < K; ++k)
#pragma unroll
        for (int j = 0; j < V; ++j) wv[k][j] = __bfloat162float(w[(c + j) * K + k]);
    }
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < V; ++j) dwacc[k][j] = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) dbacc[j] = bv[j] = 0.f;
    if (bias) ld4(bias + c, bv);
    const int lchunks = (L + CONV_BTL - 1) / CONV_BTL;
    const int nchunks = B * lchunks;
    for (int ch = blockIdx.y * 8 + sub; ch < nchunks; ch += gridDim.y * 8) {
      const int b = ch / lchunks, l0 = (ch % lchunks) * CONV_BTL;
      const int lend = min(l0 + CONV_BTL, L);
      float xh[K][V], dph[K][V];
#pragma unroll
      for (int i = 0; i < K; ++i)
#pragma unroll
        for (int j = 0; j < V; ++j) xh[i][j] = dph[i][j] = 0.f;
#pragma unroll
      for (int i = 1; i < K; ++i) {
        const int ls = l0 - K + i;
        if (ls >= 0) ld4(x + ((long long)b * L + ls) * xld + c, xh[i]);
        else if (prev) ld4(prev + ((long long)b * (K - 1) + (K - 1 + ls)) * C + c, xh[i]);
      }
#pragma unroll 4
      for (int l = l0; l < lend + K - 1; ++l) {
#pragma unroll
        for (int i = 0; i + 1 < K; ++i)
#pragma unroll
          for (int j = 0; j < V; ++j) {
            xh[i][j] = xh[i + 1][j];
            dph[i][j] = dph[i + 1][j];
          }
        if (l < L) {
          ld4(x + ((long long)b * L + l) * xld + c, xh[K - 1]);
          ld4(dy + ((long long)b * L + l) * C + c, dph[K - 1]);
          if (act) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
              float pre = bv[j];
#pragma unroll
              for (int k = 0; k < K; ++k) pre += xh[k][j] * wv[k][j];
              dph[K - 1][j] *= silu_grad(pre);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < V; ++j) xh[K - 1][j] = dph[K - 1][j] = 0.f;
        }
        if (l < lend) {   // this run's own rows: dw[k] += dpre[l] x[l-(K-1)+k], db += dpre[l]
#pragma unroll
          for (int j = 0; j < V; ++j) {
            dbacc[j] += dph[K - 1][j];
#pragma unroll
            for (int k = 0; k < K; ++k) dwacc[k][j] += dph[K - 1][j] * xh[k][j];
          }
        }
        const int lo = l - (K - 1);   // dx[lo] = sum_k w[k] dpre[lo + (K-1) - k]
        if (lo >= l0) {
          float dxa[V];
#pragma unroll
          for (int j = 0; j < V; ++j) {
            float a = 0.f;
#pragma unroll
            for (int k = 0; k < K; ++k) a += wv[k][j] * dph[K - 1 - k][j];
            dxa[j] = a;
          }
          st4(dx + ((long long)b * L + lo) * C + c, dxa);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
#pragma unroll
      for (int k = 0; k < K; ++k) atomicAdd(&s_acc[lane][k * V + j], dwacc[k][j]);
      atomicAdd(&s_acc[lane][K * V + j], dbacc[j]);
    }
  }
  __syncthreads();
  // partial layout: [part][(K+1) * C]: dw as [c][k] flattened (C*K) then db (C)
  float* pp = partial + (long long)blockIdx.y * (K + 1) * C;
  for (int i = threadIdx.x; i < 32 * (K + 1) * V; i += 256) {
    const int ln = i / ((K + 1) * V), r = i % ((K + 1) * V);
    const int k = r / V, j = r % V;
    const int cc = (blockIdx.x * 32 + ln) * V + j;
    if (cc >= C) continue;
    if (k < K) pp[(long long)cc * K + k] = s_acc[ln][r];
    else pp[(long long)C * K + cc] = s_acc[ln][r];
  }
}

// out must be zero: blockIdx.y owns every gridDim.y-th partial row and adds its sum with one atomic per element.
__global__ void conv1d_reduce_partials(const float* __restrict__ part, int nparts, int n, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
#pragma unroll 4
  for (int p = blockIdx.y; p < nparts; p += gridDim.y) s += part[(long long)p * n + i];
  atomicAdd(out + i, s);
}

}  // namespace sx
using namespace sx;

extern "C" int sx_conv1d_fwd(const void* x, const void* prev, const void* w, const void* bias, void* y, void* state_out,
                             int B, int L, int C, int K, int act, long long xld, cudaStream_t st) {
  if (C % 8 || K > CONV_MAXK || K < 1 || xld % 8 || xld < C) return -1;
  const long long total = (long long)B * ((L + CONV_TL - 1) / CONV_TL) * (C / 8);
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define SX_CONV_FWD(KK)                                                                                          \
  conv1d_fwd_kernel<KK><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)prev,              \
                                                (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, \
                                                (__nv_bfloat16*)state_out, B, L, C, act, xld)
  switch (K) {
    case 1: SX_CONV_FWD(1); break;
    case 2: SX_CONV_FWD(2); break;
    case 3: SX_CONV_FWD(3); break;
    default: SX_CONV_FWD(4); break;
  }
#undef SX_CONV_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Number of partial rows the backward kernel writes for B sequences of L tokens.
extern "C" int sx_conv1d_bwd_parts(int B, int L) {
  // four runs per warp (32 per CTA): the per-CTA prologue (taps, bias) and epilogue (partial row) cost about as much
  // as one run
  const long long chunks = (long long)B * ((L + CONV_BTL - 1) / CONV_BTL);
  const long long p = (chunks + 31) / 32;
  return (int)(p < 1 ? 1 : (p > 512 ? 512 : p));
}

// partial: scratch of sx_conv1d_bwd_parts(B, L) * (K+1) * C floats; dwdb: fp32 [(K+1)*C] = dw [C][K] then db [C].
extern "C" int sx_conv1d_bwd(const void* dy, const void* x, const void* prev, const void* w, const void* bias, void* dx,
                             float* partial, float* dwdb, int B, int L, int C, int K, int act, long long xld,
                             cudaStream_t st) {
  if (C % 8 || K > CONV_MAXK || K < 1 || xld % 8 || xld < C) return -1;
  if ((long long)B * L == 0) return 0;
  const int parts = sx_conv1d_bwd_parts(B, L);
  const dim3 grid((C / CONV_BV + 31) / 32, parts);
#define SX_CONV_BWD(KK)                                                                                          \
  conv1d_bwd_kernel<KK><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,                  \
                                              (const __nv_bfloat16*)prev, (const __nv_bfloat16*)w,                \
                                              (const __nv_bfloat16*)bias, (__nv_bfloat16*)dx, partial, B, L, C, act, xld)
  switch (K) {
    case 1: SX_CONV_BWD(1); break;
    case 2: SX_CONV_BWD(2); break;
    case 3: SX_CONV_BWD(3); break;
    default: SX_CONV_BWD(4); break;
  }
#undef SX_CONV_BWD
  const int n = (K + 1) * C;
  cudaMemsetAsync(dwdb, 0, sizeof(float) * n, st);
  conv1d_reduce_partials<<<dim3((n + 255) / 256, parts < 8 ? parts : 8), 256, 0, st>>>(partial, parts, n, dwdb);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
