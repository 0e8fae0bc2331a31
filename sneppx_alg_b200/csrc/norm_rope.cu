// N1: RMSNorm forward/backward with the residual add fused in, and LayerNorm forward.
// R1: rotary position embedding (rotate-half and adjacent-pair conventions), in place on the
//     fused QKV activation, forward and backward.
// SwiGLU / GeGLU gating forward and backward.
// All bf16 in/out with fp32 math; rows are read with 128-bit loads. These replace the
// reference's layernorm / rmsnorm / rope kernels (kernel/cuda/tensor_cuda.cu:393-441,
// kernel/cuda/autodiff_cuda.cu:444-487, kernel/cuda/attention_cuda.cu:895-943) and the CPU gated
// activations (kernel/activations/gated_activations.c:33-118).
#include "common.cuh"
#include "sx_api.h"

namespace sx {

// y = rmsnorm(x + res_in) * w ; res_out = x + res_in ; rstd saved for backward.
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ res_in,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y,
                                                          __nv_bfloat16* __restrict__ res_out,
                                                          float* __restrict__ rstd, int d, float eps) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may start its prologue
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * d;
  const int nvec = d >> 3;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    unpack8(ld8(xr + i * 8), f);
    if (res_in) {
      float g[8];
      unpack8(ld8(res_in + row * d + i * 8), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      // round through bf16 so that the statistics match what backward will re-read
      bf16x8 hp = pack8(f);
      unpack8(hp, f);
      if (res_out) st8(res_out + row * d + i * 8, hp);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const __nv_bfloat16* hr = (res_in && res_out) ? res_out + row * d : xr;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8], g[8];
    unpack8(ld8(hr + i * 8), f);
    if (res_in && !res_out) {
      unpack8(ld8(res_in + row * d + i * 8), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
    }
    unpack8(ld8(w + i * 8), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * g[j];
    st8(y + row * d + i * 8, pack8(f));
  }
}

// dx = rstd * (w*dy) - h * rstd^3 * mean(w*dy*h) (+ dres) ; dw partial sums per CTA.
// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its dw partials in
// registers (thread t owns column vectors t, t + blockDim, ...; at most MAXV of them).
template <int MAXV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ h,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rstd,
                                                          const __nv_bfloat16* __restrict__ dres,
                                                          __nv_bfloat16* __restrict__ dx,
                                                          float* __restrict__ dw_partial, int T, int d) {
  __shared__ float red[33];
  const int nvec = d >> 3;
  float acc[MAXV][8];
  float wv[MAXV][8];
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[k][j] = 0.f;
    if (i < nvec) unpack8(ld8(w + i * 8), wv[k]);
  }
  for (long long row = blockIdx.x; row < T; row += gridDim.x) {
    const float r = rstd[row];
    float dot = 0.f;
    float g[MAXV][8], hv[MAXV][8];
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        unpack8(ld8(dy + row * d + i * 8), g[k]);
        unpack8(ld8(h + row * d + i * 8), hv[k]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[k][j] += g[k][j] * hv[k][j] * r;
          g[k][j] *= wv[k][j];
          dot += g[k][j] * hv[k][j];
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * r * r * r / d;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = g[k][j] * r - hv[k][j] * c;
        if (dres) {
          float e[8];
          unpack8(ld8(dres + row * d + i * 8), e);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += e[j];
        }
        st8(dx + row * d + i * 8, pack8(o));
      }
    }
  }
#pragma unroll
  for (int k = 0; k < MAXV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float* o = dw_partial + (long long)blockIdx.x * d + i * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = acc[k][j];
    }
  }
}

__global__ void colsum_partials_kernel(const float* __restrict__ part, int nparts, int d,
                                       __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32,
                                       int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += part[(long long)p * d + c];
  if (out_f32) out_f32[c] = accumulate ? out_f32[c] + s : s;
  if (out_bf16) out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + s : s);
}

__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ b,
                                                            __nv_bfloat16* __restrict__ y, float* __restrict__ mean,
                                                            float* __restrict__ rstd, int d, float eps) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) s += __bfloat162float(x[row * d + i]);
  const float mu = block_sum(s, red) / d;
  float v = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float t = __bfloat162float(x[row * d + i]) - mu;
    v += t * t;
  }
  const float r = rsqrtf(block_sum(v, red) / d + eps);
  if (threadIdx.x == 0) {
    if (mean) mean[row] = mu;
    if (rstd) rstd[row] = r;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float t = (__bfloat162float(x[row * d + i]) - mu) * r * __bfloat162float(w[i]);
    if (b) t += __bfloat162float(b[i]);
    y[row * d + i] = __float2bfloat16(t);
  }
}

// RoPE in place. x: [tokens, row_stride] with `heads` heads of size D starting at column 0.
// table: [max_pos, D/2] cos and sin (fp32). pos: optional per-token position, else token % seq.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, long long tokens,
                            int seq, int heads, int D, long long row_stride, int interleaved, float sign) {
  const int half = D >> 1;
  const long long total = tokens * heads * half;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = idx % half;
    const int hd = (idx / half) % heads;
    const long long t = idx / ((long long)half * heads);
    const int p = pos ? pos[t] : (int)(t % seq);
    const float c = cos_t[(long long)p * half + i];
    const float s = sin_t[(long long)p * half + i] * sign;
    __nv_bfloat16* base = x + t * row_stride + (long long)hd * D;
    const int i1 = interleaved ? 2 * i : i;
    const int i2 = interleaved ? 2 * i + 1 : i + half;
    const float a = __bfloat162float(base[i1]);
    const float b = __bfloat162float(base[i2]);
    base[i1] = __float2bfloat16(a * c - b * s);
    base[i2] = __float2bfloat16(b * c + a * s);
  }
}

// Rotate-half layout, 8 rotation pairs per thread: two 16-byte loads of x (the halves), 2 x 32 bytes of cos / sin.
__global__ void rope_vec8_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                                 const float* __restrict__ sin_t, const int* __restrict__ pos, long long tokens,
                                 int seq, int heads, int D, long long row_stride, float sign) {
  const int half = D >> 1, hv = half >> 3;
  const long long total = tokens * heads * hv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int i = (int)(idx % hv) * 8;
    const long long th = idx / hv;
    const int hd = (int)(th % heads);
    const long long t = th / heads;
    const int p = pos ? pos[t] : (int)(t % seq);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)p * half + i);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)p * half + i);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    __nv_bfloat16* base = x + t * row_stride + (long long)hd * D + i;
    float a[8], b[8];
    unpack8(ld8(base), a);
    unpack8(ld8(base + half), b);
    float ra[8], rb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = sn[j] * sign;
      ra[j] = a[j] * c[j] - b[j] * s;
      rb[j] = b[j] * c[j] + a[j] * s;
    }
    st8(base, pack8(ra));
    st8(base + half, pack8(rb));
  }
}

// h = act(gate) * up ; gu = [T, 2F] (gate | up). act: 0 silu (SwiGLU), 1 gelu (GeGLU), 2 relu (ReGLU)
__device__ __forceinline__ float gate_act(float g, int act) {
  if (act == 0) return g / (1.f + __expf(-g));
  if (act == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
  }
  return fmaxf(g, 0.f);
}
__device__ __forceinline__ float gate_act_grad(float g, int act) {
  if (act == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (act == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float u = k0 * (g + k1 * g * g * g);
    const float th = tanhf(u);
    return 0.5f * (1.f + th) + 0.5f * g * (1.f - th * th) * k0 * (1.f + 3.f * k1 * g * g);
  }
  return g > 0.f ? 1.f : 0.f;
}

__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long T,
                               int F, int act) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a dependent launch may start its prologue
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / fv;
    const int c = (idx % fv) * 8;
    float g[8], u[8];
    unpack8(ld8(gu + t * 2 * F + c), g);
    unpack8(ld8(gu + t * 2 * F + F + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = gate_act(g[j], act) * u[j];
    st8(h + t * F + c, pack8(g));
  }
}

__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu,
                               __nv_bfloat16* __restrict__ dgu, long long T, int F, int act) {
  const int fv = F >> 3;
  const long long total = T * fv;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / fv;
    const int c = (idx % fv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld8(gu + t * 2 * F + c), g);
    unpack8(ld8(gu + t * 2 * F + F + c), u);
    unpack8(ld8(dh + t * F + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * gate_act_grad(g[j], act);
      du[j] = d[j] * gate_act(g[j], act);
    }
    st8(dgu + t * 2 * F + c, pack8(dg));
    st8(dgu + t * 2 * F + F + c, pack8(du));
  }
}

}  // namespace sx

using namespace sx;

extern "C" int sx_rmsnorm_fwd(const void* x, const void* res_in, const void* w, void* y, void* res_out, float* rstd,
                              long long T, int d, float eps, cudaStream_t st) {
  if (d % 8) return -1;
  if (T == 0) return 0;
  rmsnorm_fwd_kernel<<<(unsigned)T, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res_in,
                                                  (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                                  (__nv_bfloat16*)res_out, rstd, d, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// dw_partial: scratch of nparts*d floats (nparts = value returned by sx_rmsnorm_bwd_parts()).
extern "C" int sx_rmsnorm_bwd_parts() { return 296; }

extern "C" int sx_rmsnorm_bwd(const void* dy, const void* h, const void* w, const float* rstd, const void* dres,
                              void* dx, float* dw_partial, void* dw_bf16, float* dw_f32, int accumulate, long long T,
                              int d, cudaStream_t st) {
  if (d % 8) return -1;
  if (T == 0) return 0;
  const int parts = sx_rmsnorm_bwd_parts();
  const int nvec = d / 8;
  const int need = (nvec + 255) / 256;
  auto args = [&](auto kern) {
    kern<<<parts, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w, rstd,
                                (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dw_partial, (int)T, d);
  };
  if (need <= 1) args(rmsnorm_bwd_kernel<1>);
  else if (need <= 2) args(rmsnorm_bwd_kernel<2>);
  else if (need <= 4) args(rmsnorm_bwd_kernel<4>);
  else if (need <= 8) args(rmsnorm_bwd_kernel<8>);
  else return -2;
  colsum_partials_kernel<<<(d + 255) / 256, 256, 0, st>>>(dw_partial, parts, d, (__nv_bfloat16*)dw_bf16, dw_f32,
                                                          accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                                long long T, int d, float eps, cudaStream_t st) {
  if (T == 0) return 0;
  layernorm_fwd_kernel<<<(unsigned)T, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                    (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, d, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_rope(void* x, const float* cos_t, const float* sin_t, const int* pos, long long tokens, int seq,
                       int heads, int D, long long row_stride, int interleaved, int backward, cudaStream_t st) {
  if (tokens == 0) return 0;
  if (!interleaved && (D / 2) % 8 == 0 && row_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 && (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0) {
    const long long tv = tokens * heads * (D / 16);
    const int bv = (int)((tv + 255) / 256 < 148 * 16 ? (tv + 255) / 256 : 148 * 16);
    rope_vec8_kernel<<<bv, 256, 0, st>>>((__nv_bfloat16*)x, cos_t, sin_t, pos, tokens, seq, heads, D, row_stride,
                                         backward ? -1.f : 1.f);
    return cudaGetLastError() == cudaSuccess ? 0 : -11;
  }
  const long long total = tokens * heads * (D / 2);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  rope_kernel<<<blocks, 256, 0, st>>>((__nv_bfloat16*)x, cos_t, sin_t, pos, tokens, seq, heads, D, row_stride,
                                      interleaved, backward ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_glu_fwd(const void* gu, void* h, long long T, int F, int act, cudaStream_t st) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  const long long total = T * (F / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  glu_fwd_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)h, T, F, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_glu_bwd(const void* dh, const void* gu, void* dgu, long long T, int F, int act, cudaStream_t st) {
  if (F % 8) return -1;
  if (T == 0) return 0;
  const long long total = T * (F / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  glu_bwd_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T,
                                         F, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
