// Counter-based RNG (Philox4x32-10) fills, fused dropout that regenerates its mask in backward, LayerNorm backward,
// gradient compression (block int8, block top-2), weighted federated average, and adversarial-robustness elementwise
// steps (FGSM, PGD projection, sine obfuscation, Gaussian smoothing).
//
// Reference counterparts: kernel/cuda/rng_cuda.cu (Philox state per thread via cuRAND, uniform / normal / bernoulli,
// fused dropout :418), kernel/cuda/autodiff_cuda.cu:331-431 (LayerNorm backward), algorithms/fm/cuda/fm_cuda.cu:100-240
// (int8 gradient quantisation, block top-2 sparsify, weighted average), algorithms/arc/cuda/arc_cuda.cu:22-140.
// All of these are bandwidth-bound: every thread moves 16-byte vectors, and random numbers are a pure function of
// (seed, element index), so no generator state is stored and a dropout mask never touches memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sx_api.h"

namespace sx {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// four random words for elements [4 * q, 4 * q + 4) of stream `offset`
__device__ __forceinline__ uint4 rand4(unsigned long long seed, unsigned long long offset, unsigned long long q) {
  return philox4x32_10(make_uint4((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)),
                       make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
}

__device__ __forceinline__ float u01(uint32_t r) { return ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f); }  // (0, 1)

__device__ __forceinline__ void normal4(uint4 r, float* z) {
  float a0 = sqrtf(-2.0f * __logf(u01(r.x))), a1 = sqrtf(-2.0f * __logf(u01(r.z)));
  float s0, c0, s1, c1;
  __sincosf(6.283185307179586f * u01(r.y), &s0, &c0);
  __sincosf(6.283185307179586f * u01(r.w), &s1, &c1);
  z[0] = a0 * c0; z[1] = a0 * s0; z[2] = a1 * c1; z[3] = a1 * s1;
}

// mode 0: uniform in [lo, hi); 1: normal(mean = lo, std = hi); 2: bernoulli(p = lo) as 0 / 1
__global__ void __launch_bounds__(256) rng_fill_kernel(float* out, long long n, int mode, float lo, float hi,
                                                        unsigned long long seed, unsigned long long offset) {
  long long nq = (n + 3) / 4;
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < nq; q += (long long)gridDim.x * blockDim.x) {
    uint4 r = rand4(seed, offset, (unsigned long long)q);
    float v[4];
    if (mode == 1) { normal4(r, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = lo + hi * v[i];
    } else {
      uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = mode == 0 ? lo + (hi - lo) * u01(w[i]) : (u01(w[i]) < lo ? 1.0f : 0.0f);
    }
    if (4 * q + 4 <= n) *reinterpret_cast<float4*>(out + 4 * q) = make_float4(v[0], v[1], v[2], v[3]);
    else for (int i = 0; 4 * q + i < n; ++i) out[4 * q + i] = v[i];
  }
}

// y = x * keep / (1 - p) with keep = (u >= p); the same call with x = dy is the backward pass. n % 8 == 0.
// Two 16-byte vectors are in flight per thread and iteration.
__device__ __forceinline__ uint4 dropout8(uint4 raw, unsigned long long v, float p, float scale, unsigned long long seed, unsigned long long offset) {
  uint4 r0 = rand4(seed, offset, 2ull * v), r1 = rand4(seed, offset, 2ull * v + 1);
  uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
  __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
  for (int i = 0; i < 8; ++i) e[i] = __float2bfloat16(u01(w[i]) >= p ? __bfloat162float(e[i]) * scale : 0.0f);
  return raw;
}

__global__ void __launch_bounds__(256) dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                       long long n, float p, unsigned long long seed, unsigned long long offset) {
  const float scale = 1.0f / (1.0f - p);
  const long long nv = n / 8, stride = (long long)gridDim.x * blockDim.x;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nv; v += 2 * stride) {
    const long long v2 = v + stride;
    uint4 a = *reinterpret_cast<const uint4*>(x + 8 * v), b = make_uint4(0, 0, 0, 0);
    if (v2 < nv) b = *reinterpret_cast<const uint4*>(x + 8 * v2);
    *reinterpret_cast<uint4*>(y + 8 * v) = dropout8(a, (unsigned long long)v, p, scale, seed, offset);
    if (v2 < nv) *reinterpret_cast<uint4*>(y + 8 * v2) = dropout8(b, (unsigned long long)v2, p, scale, seed, offset);
  }
}

// LayerNorm backward. A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; thread t owns column vectors t,
// t + 256, ... (at most MAXV of them), so x and dy are read once, and dgamma / dbeta accumulate in registers across
// the CTA's rows. mean / rstd come from the forward pass. Each CTA writes one [2, cols] slab of partial sums.
template <int MAXV>
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                             const float* __restrict__ gamma, const float* __restrict__ mean,
                                                             const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                                             float* __restrict__ partials, long long rows, int cols) {
  __shared__ float red[2][8];
  const int nvec = cols >> 3, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float acc_g[MAXV][8], acc_b[MAXV][8], gm[MAXV][8];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * 256;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc_g[k][j] = 0.f; acc_b[k][j] = 0.f; gm[k][j] = i < nvec ? gamma[i * 8 + j] : 0.f; }
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const float mu = mean[row], rs = rstd[row];
    float xh[MAXV][8], gg[MAXV][8], a = 0.f, b = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        uint4 rx = *reinterpret_cast<const uint4*>(x + row * cols + i * 8), rg = *reinterpret_cast<const uint4*>(dy + row * cols + i * 8);
        const __nv_bfloat16 *ex = reinterpret_cast<const __nv_bfloat16*>(&rx), *eg = reinterpret_cast<const __nv_bfloat16*>(&rg);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float g = __bfloat162float(eg[j]);
          xh[k][j] = (__bfloat162float(ex[j]) - mu) * rs;
          acc_g[k][j] += g * xh[k][j];
          acc_b[k][j] += g;
          gg[k][j] = g * gm[k][j];
          a += gg[k][j];
          b += gg[k][j] * xh[k][j];
        }
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    __syncthreads();  // the previous row's readers are done with `red`
    if (lane == 0) { red[0][warp] = a; red[1][warp] = b; }
    __syncthreads();
    a = 0.f; b = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
    a /= cols; b /= cols;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * 256;
      if (i < nvec) {
        uint4 ro;
        __nv_bfloat16* eo = reinterpret_cast<__nv_bfloat16*>(&ro);
#pragma unroll
        for (int j = 0; j < 8; ++j) eo[j] = __float2bfloat16(rs * (gg[k][j] - a - xh[k][j] * b));
        *reinterpret_cast<uint4*>(dx + row * cols + i * 8) = ro;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * 256;
    if (i < nvec) {
      float* o = partials + (long long)blockIdx.x * 2 * cols + i * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = acc_g[k][j]; o[cols + j] = acc_b[k][j]; }
    }
  }
}

// out[2, cols] = sum over `nblk` slabs
__global__ void __launch_bounds__(256) ln_reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out, int nblk, int cols2) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols2) return;
  float s = 0;
  for (int b = 0; b < nblk; ++b) s += partials[(long long)b * cols2 + c];
  out[c] = s;
}

}  // namespace sx

namespace sx {

// ---- gradient compression and federated averaging (fp32) -----------------------------------------------------
// One warp per block of 256 values: scale = absmax / 127, q = round(x / scale). n % 256 == 0.
__global__ void __launch_bounds__(256) fm_quant_int8_kernel(const float* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ scales, long long nblocks) {
  const int lane = threadIdx.x & 31;
  for (long long b = blockIdx.x * 8ll + (threadIdx.x >> 5); b < nblocks; b += gridDim.x * 8ll) {
    const float4* src = reinterpret_cast<const float4*>(x + b * 256 + lane * 8);
    float4 v0 = src[0], v1 = src[1];
    float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float m = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = m / 127.0f, inv = m > 0 ? 127.0f / m : 0.0f;
    if (lane == 0) scales[b] = scale;
    int8_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = (int8_t)max(-127, min(127, __float2int_rn(v[i] * inv)));
    *reinterpret_cast<uint2*>(q + b * 256 + lane * 8) = *reinterpret_cast<uint2*>(out);
  }
}

__global__ void __launch_bounds__(256) fm_dequant_int8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, float* __restrict__ y, long long nblocks) {
  const int lane = threadIdx.x & 31;
  for (long long b = blockIdx.x * 8ll + (threadIdx.x >> 5); b < nblocks; b += gridDim.x * 8ll) {
    uint2 raw = *reinterpret_cast<const uint2*>(q + b * 256 + lane * 8);
    const int8_t* e = reinterpret_cast<const int8_t*>(&raw);
    const float s = scales[b];
    float4* dst = reinterpret_cast<float4*>(y + b * 256 + lane * 8);
    dst[0] = make_float4(e[0] * s, e[1] * s, e[2] * s, e[3] * s);
    dst[1] = make_float4(e[4] * s, e[5] * s, e[6] * s, e[7] * s);
  }
}

// Per block of 32 values keep the two of largest magnitude (lowest index wins ties); `residual` (optional) receives
// what was dropped, the error-feedback term that the caller adds to the next gradient. n % 32 == 0.
__global__ void __launch_bounds__(256) fm_block_top2_kernel(const float* __restrict__ x, float* __restrict__ kept, float* __restrict__ residual, long long nblocks) {
  const int lane = threadIdx.x & 31;
  const long long wstride = gridDim.x * 8ll;
  for (long long b0 = blockIdx.x * 8ll + (threadIdx.x >> 5); b0 < nblocks; b0 += 4 * wstride) {
    float vals[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) { const long long b = b0 + u * wstride; vals[u] = b < nblocks ? x[b * 32 + lane] : 0.0f; }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long b = b0 + u * wstride;
      if (b >= nblocks) break;
      const float v = vals[u], a = fabsf(v);
      int first = -1, second = -1;
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        float m = (lane == first) ? -1.0f : a;
        int idx = lane;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          float om = __shfl_xor_sync(0xffffffffu, m, o);
          int oi = __shfl_xor_sync(0xffffffffu, idx, o);
          if (om > m || (om == m && oi < idx)) { m = om; idx = oi; }
        }
        if (pass == 0) first = idx; else second = idx;
      }
      const bool keep = lane == first || lane == second;
      kept[b * 32 + lane] = keep ? v : 0.0f;
      if (residual) residual[b * 32 + lane] = keep ? 0.0f : v;
    }
  }
}

struct FmAvgArgs { const float* in[16]; float w[16]; int count; };

__global__ void __launch_bounds__(256) fm_weighted_avg_kernel(FmAvgArgs a, float* __restrict__ out, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0, 0, 0, 0);
    for (int k = 0; k < a.count; ++k) {
      float4 v = reinterpret_cast<const float4*>(a.in[k])[i];
      acc.x += a.w[k] * v.x; acc.y += a.w[k] * v.y; acc.z += a.w[k] * v.z; acc.w += a.w[k] * v.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
}

// ---- adversarial-robustness steps (fp32, n % 4 == 0) ---------------------------------------------------------------
// mode 0 FGSM:   out = clamp(x + eps * sign(g), lo, hi)
// mode 1 PGD:    out = clamp(clip(x + alpha * sign(g), x0 - eps, x0 + eps), lo, hi)
// mode 2 sine obfuscation of a gradient: out = x + eps * sin(100 x)
// mode 3 Gaussian smoothing sample: out = x + eps * N(0, 1)
__global__ void __launch_bounds__(256) arc_step_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ x0,
                                                        float* __restrict__ out, long long n4, int mode, float eps, float alpha, float lo, float hi,
                                                        unsigned long long seed, unsigned long long offset) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 xv = reinterpret_cast<const float4*>(x)[i];
    float v[4] = {xv.x, xv.y, xv.z, xv.w}, r[4];
    if (mode == 0 || mode == 1) {
      float4 gv = reinterpret_cast<const float4*>(g)[i];
      float gg[4] = {gv.x, gv.y, gv.z, gv.w};
      float c[4] = {0, 0, 0, 0};
      if (mode == 1) { float4 cv = reinterpret_cast<const float4*>(x0)[i]; c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w; }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float sgn = gg[k] > 0 ? 1.0f : (gg[k] < 0 ? -1.0f : 0.0f);
        float t = v[k] + (mode == 0 ? eps : alpha) * sgn;
        if (mode == 1) t = fminf(fmaxf(t, c[k] - eps), c[k] + eps);
        r[k] = fminf(fmaxf(t, lo), hi);
      }
    } else if (mode == 2) {
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = v[k] + eps * sinf(100.0f * v[k]);
    } else {
      float z[4];
      normal4(rand4(seed, offset, (unsigned long long)i), z);
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = v[k] + eps * z[k];
    }
    reinterpret_cast<float4*>(out)[i] = make_float4(r[0], r[1], r[2], r[3]);
  }
}

static inline int grid_for(long long work_items, int per_block) {
  long long g = (work_items + per_block - 1) / per_block;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

}  // namespace sx

extern "C" {

int sx_rng_fill(float* out, long long n, int mode, float a, float b, unsigned long long seed, unsigned long long offset, cudaStream_t st) {
  if (n <= 0 || mode < 0 || mode > 2 || ((uintptr_t)out & 15)) return -1;
  sx::rng_fill_kernel<<<sx::grid_for((n + 3) / 4, 256), 256, 0, st>>>(out, n, mode, a, b, seed, offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, unsigned long long offset, cudaStream_t st) {
  if (n <= 0 || n % 8 || p < 0.0f || p >= 1.0f || (((uintptr_t)x | (uintptr_t)y) & 15)) return -1;
  sx::dropout_kernel<<<sx::grid_for(n / 8, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p, seed, offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_layernorm_bwd_blocks(long long rows) { return (int)(rows < 148 * 4 ? (rows < 1 ? 1 : rows) : 148 * 4); }

// mean, rstd: [rows] fp32 from sx_layernorm_fwd. partials: [sx_layernorm_bwd_blocks(rows), 2, cols] fp32 scratch;
// dgamma_dbeta: [2, cols] (row 0 dgamma, row 1 dbeta). cols % 8 == 0, cols <= 8192.
int sx_layernorm_bwd(const void* x, const void* dy, const float* gamma, const float* mean, const float* rstd, void* dx,
                     float* partials, float* dgamma_dbeta, long long rows, int cols, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || cols % 8 || cols > 8192) return -1;
  const int nblk = sx_layernorm_bwd_blocks(rows), need = (cols / 8 + 255) / 256;
  auto go = [&](auto kern) {
    kern<<<nblk, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, gamma, mean, rstd, (__nv_bfloat16*)dx, partials, rows, cols);
  };
  if (need <= 1) go(sx::layernorm_bwd_kernel<1>);
  else if (need <= 2) go(sx::layernorm_bwd_kernel<2>);
  else go(sx::layernorm_bwd_kernel<4>);
  sx::ln_reduce_partials_kernel<<<(2 * cols + 255) / 256, 256, 0, st>>>(partials, dgamma_dbeta, nblk, 2 * cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_fm_quant_int8(const float* x, void* q, float* scales, long long n, cudaStream_t st) {
  if (n <= 0 || n % 256) return -1;
  sx::fm_quant_int8_kernel<<<sx::grid_for(n / 256, 8), 256, 0, st>>>(x, (int8_t*)q, scales, n / 256);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_fm_dequant_int8(const void* q, const float* scales, float* y, long long n, cudaStream_t st) {
  if (n <= 0 || n % 256) return -1;
  sx::fm_dequant_int8_kernel<<<sx::grid_for(n / 256, 8), 256, 0, st>>>((const int8_t*)q, scales, y, n / 256);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_fm_block_top2(const float* x, float* kept, float* residual, long long n, cudaStream_t st) {
  if (n <= 0 || n % 32) return -1;
  sx::fm_block_top2_kernel<<<sx::grid_for(n / 32, 8), 256, 0, st>>>(x, kept, residual, n / 32);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_fm_weighted_avg(const float* const* inputs, const float* weights, int count, float* out, long long n, cudaStream_t st) {
  if (count < 1 || count > 16 || n <= 0 || n % 4) return -1;
  sx::FmAvgArgs a;
  for (int i = 0; i < count; ++i) { a.in[i] = inputs[i]; a.w[i] = weights[i]; }
  a.count = count;
  sx::fm_weighted_avg_kernel<<<sx::grid_for(n / 4, 256), 256, 0, st>>>(a, out, n / 4);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int sx_arc_step(const float* x, const float* g, const float* x0, float* out, long long n, int mode, float eps, float alpha,
                float lo, float hi, unsigned long long seed, unsigned long long offset, cudaStream_t st) {
  if (n <= 0 || n % 4 || mode < 0 || mode > 3 || (mode <= 1 && !g) || (mode == 1 && !x0)) return -1;
  sx::arc_step_kernel<<<sx::grid_for(n / 4, 256), 256, 0, st>>>(x, g, x0, out, n / 4, mode, eps, alpha, lo, hi, seed, offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
