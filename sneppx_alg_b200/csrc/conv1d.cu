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
                                                         int act) {
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
      if (ls >= 0) unpack8(ld8(x + ((long long)b * L + ls) * C + c), hist[i]);
      else if (prev) unpack8(ld8(prev + ((long long)b * (K - 1) + (K - 1 + ls)) * C + c), hist[i]);
    }
    const int l1 = min(L, l0 + CONV_TL);
    for (int l = l0; l < l1; ++l) {
      const bf16x8 raw = ld8(x + ((long long)b * L + l) * C + c);
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

// dx and per-CTA partials of dw / dbias. Each CTA owns a contiguous range of (b, l) rows and all channels;
// thread t owns channel vectors t, t + blockDim, ... (C/8 <= blockDim * CONV_VEC).
constexpr int CONV_VEC = 4;
__global__ void __launch_bounds__(256) conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                         const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ prev,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ bias,
                                                         __nv_bfloat16* __restrict__ dx, float* __restrict__ partial,
                                                         int B, int L, int C, int K, int act, int rows_per_cta) {
  const int cv = C >> 3;
  const long long rows = (long long)B * L;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  for (int vi = 0; vi < CONV_VEC; ++vi) {
    const int v = threadIdx.x + vi * blockDim.x;
    if (v >= cv) break;
    const int c = v * 8;
    float wv[CONV_MAXK][8], bv[8];
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[k][j] = __bfloat162float(w[(c + j) * K + k]);
#pragma unroll
    for (int j = 0; j < 8; ++j) bv[j] = bias ? __bfloat162float(bias[c + j]) : 0.f;
    float dwacc[CONV_MAXK][8], dbacc[8];
    for (int k = 0; k < CONV_MAXK; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) dwacc[k][j] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) dbacc[j] = 0.f;
    auto load_x = [&](int b, int ls, float (&o)[8]) {
      if (ls >= 0) unpack8(ld8(x + ((long long)b * L + ls) * C + c), o);
      else if (prev) unpack8(ld8(prev + ((long long)b * (K - 1) + (K - 1 + ls)) * C + c), o);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = 0.f;
      }
    };
    // dpre at row (b, l) = dy * act'(pre); recompute pre from x
    auto dpre_at = [&](int b, int l, float (&o)[8]) {
      unpack8(ld8(dy + ((long long)b * L + l) * C + c), o);
      if (act) {
        float pre[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) pre[j] = bv[j];
        for (int k = 0; k < K; ++k) {
          float xv[8];
          load_x(b, l - (K - 1) + k, xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) pre[j] += xv[j] * wv[k][j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= silu_grad(pre[j]);
      }
    };
    for (long long r = r0; r < r1; ++r) {
      const int l = r % L, b = r / L;
      // dx[l] = sum_k w[k] * dpre[l + (K-1) - k]
      float dxa[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) dxa[j] = 0.f;
      for (int k = 0; k < K; ++k) {
        const int lo = l + (K - 1) - k;
        if (lo >= L) continue;
        float dp[8];
        dpre_at(b, lo, dp);
#pragma unroll
        for (int j = 0; j < 8; ++j) dxa[j] += wv[k][j] * dp[j];
      }
      st8(dx + r * C + c, pack8(dxa));
      // dw[k] += dpre[l] * x[l - (K-1) + k] ; db += dpre[l]
      float dp[8];
      dpre_at(b, l, dp);
#pragma unroll
      for (int j = 0; j < 8; ++j) dbacc[j] += dp[j];
      for (int k = 0; k < K; ++k) {
        float xv[8];
        load_x(b, l - (K - 1) + k, xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) dwacc[k][j] += dp[j] * xv[j];
      }
    }
    // partial layout: [cta][ (K+1) * C ] : dw as [c][k] flattened (C*K) then db (C)
    float* pp = partial + (long long)blockIdx.x * (K + 1) * C;
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) pp[(c + j) * K + k] = dwacc[k][j];
#pragma unroll
    for (int j = 0; j < 8; ++j) pp[(long long)C * K + c + j] = dbacc[j];
  }
}

__global__ void conv1d_reduce_partials(const float* __restrict__ part, int nparts, int n, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(long long)p * n + i];
  out[i] = s;
}

}  // namespace sx
using namespace sx;

extern "C" int sx_conv1d_fwd(const void* x, const void* prev, const void* w, const void* bias, void* y, void* state_out,
                             int B, int L, int C, int K, int act, cudaStream_t st) {
  if (C % 8 || K > CONV_MAXK || K < 1) return -1;
  const long long total = (long long)B * ((L + CONV_TL - 1) / CONV_TL) * (C / 8);
  if (total == 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define SX_CONV_FWD(KK)                                                                                          \
  conv1d_fwd_kernel<KK><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)prev,              \
                                                (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, \
                                                (__nv_bfloat16*)state_out, B, L, C, act)
  switch (K) {
    case 1: SX_CONV_FWD(1); break;
    case 2: SX_CONV_FWD(2); break;
    case 3: SX_CONV_FWD(3); break;
    default: SX_CONV_FWD(4); break;
  }
#undef SX_CONV_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_conv1d_bwd_parts(long long rows) {
  long long p = (rows + 63) / 64;
  return (int)(p < 1 ? 1 : (p > 592 ? 592 : p));
}

// partial: scratch of sx_conv1d_bwd_parts(B*L) * (K+1) * C floats; dwdb: fp32 [(K+1)*C] = dw [C][K] then db [C].
extern "C" int sx_conv1d_bwd(const void* dy, const void* x, const void* prev, const void* w, const void* bias, void* dx,
                             float* partial, float* dwdb, int B, int L, int C, int K, int act, cudaStream_t st) {
  if (C % 8 || K > CONV_MAXK || K < 1 || C / 8 > 256 * CONV_VEC) return -1;
  const long long rows = (long long)B * L;
  if (rows == 0) return 0;
  const int parts = sx_conv1d_bwd_parts(rows);
  const int rpc = (int)((rows + parts - 1) / parts);
  conv1d_bwd_kernel<<<parts, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                           (const __nv_bfloat16*)prev, (const __nv_bfloat16*)w,
                                           (const __nv_bfloat16*)bias, (__nv_bfloat16*)dx, partial, B, L, C, K, act,
                                           rpc);
  const int n = (K + 1) * C;
  conv1d_reduce_partials<<<(n + 255) / 256, 256, 0, st>>>(partial, parts, n, dwdb);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
