// O1: fused AdamW over flat buffers and over tensor lists (fp32 master weights + moments, bf16 or
//     fp32 gradients, optional bf16 parameter copy written in the same pass).
// O2: gradient L2 norm (deterministic two-stage reduction), non-finite flag, clip coefficient.
// Also SGD-momentum and Lion updates for the optimizer zoo.
// Update order matches the reference (bindings/python/SneppX_ALG/interface_bindings/optim.py:96-114,
// kernel/cuda/optim_cuda.cu:167-207): moments -> bias correction -> decoupled weight decay ->
// Adam step.
#include "common.cuh"
#include "sx_api.h"

namespace sx {

struct AdamHyper {
  float lr, beta1, beta2, eps, wd, bc1, bc2;  // bc = 1 - beta^t
  float grad_scale;                           // multiplies every gradient (e.g. 1/world)
};

__device__ __forceinline__ void adamw_elem(float& p, float& m, float& v, float g, const AdamHyper& h) {
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float mh = m / h.bc1;
  const float vh = v / h.bc2;
  p -= h.lr * h.wd * p;
  p -= h.lr * mh / (sqrtf(vh) + h.eps);
}

// clip: optional device scalar multiplying the gradient (written by sx_clip_coef).
template <bool G_BF16>
__global__ void __launch_bounds__(256) adamw_flat_kernel(float* __restrict__ p, float* __restrict__ m,
                                                         float* __restrict__ v, const void* __restrict__ g,
                                                         __nv_bfloat16* __restrict__ p16, long long n,
                                                         AdamHyper h, const float* __restrict__ clip) {
  const float gs = h.grad_scale * (clip ? *clip : 1.f);
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gg[4];
    if (G_BF16) {
      const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
    } else {
      const float4 t = reinterpret_cast<const float4*>(g)[i];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
    }
    adamw_elem(pp.x, mm.x, vv.x, gg[0] * gs, h);
    adamw_elem(pp.y, mm.y, vv.y, gg[1] * gs, h);
    adamw_elem(pp.z, mm.z, vv.z, gg[2] * gs, h);
    adamw_elem(pp.w, mm.w, vv.w, gg[3] * gs, h);
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(p16)[i] = o;
    }
  }
  // tail
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = (n4 << 2) + threadIdx.x;
    float pp = p[i], mm = m[i], vv = v[i];
    const float gg = G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])
                            : reinterpret_cast<const float*>(g)[i];
    adamw_elem(pp, mm, vv, gg * gs, h);
    p[i] = pp; m[i] = mm; v[i] = vv;
    if (p16) p16[i] = __float2bfloat16(pp);
  }
}

constexpr int MT_MAX = 24;
struct MultiTensorTable {
  float* p[MT_MAX];
  float* m[MT_MAX];
  float* v[MT_MAX];
  const void* g[MT_MAX];
  __nv_bfloat16* p16[MT_MAX];
  long long n[MT_MAX];
  float wd[MT_MAX];
  int count;
};

template <bool G_BF16>
__global__ void __launch_bounds__(256) adamw_multi_kernel(const __grid_constant__ MultiTensorTable tb, AdamHyper h,
                                                          const float* __restrict__ clip) {
  const int t = blockIdx.y;
  if (t >= tb.count) return;
  h.wd = tb.wd[t];
  const float gs = h.grad_scale * (clip ? *clip : 1.f);
  float* p = tb.p[t];
  float* m = tb.m[t];
  float* v = tb.v[t];
  __nv_bfloat16* p16 = tb.p16[t];
  const long long n = tb.n[t];
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float pp = p[i], mm = m[i], vv = v[i];
    const float gg = G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(tb.g[t])[i])
                            : reinterpret_cast<const float*>(tb.g[t])[i];
    adamw_elem(pp, mm, vv, gg * gs, h);
    p[i] = pp; m[i] = mm; v[i] = vv;
    if (p16) p16[i] = __float2bfloat16(pp);
  }
}

// ---- L2 norm: stage 1 writes one partial (sum of squares) per CTA into `partials`, stage 2
// adds them in index order, so the result does not depend on scheduling.
template <bool G_BF16>
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const void* __restrict__ g, long long n,
                                                            float* __restrict__ partials, int* __restrict__ nonfinite) {
  __shared__ float red[33];
  float s = 0.f;
  bool bad = false;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float x = G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i])
                           : reinterpret_cast<const float*>(g)[i];
    bad |= !isfinite(x);
    s += x * x;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
  if (bad && nonfinite) atomicExch(nonfinite, 1);
}

// out[0] (+)= sum(partials) ; when finalize: out[1] = sqrt(out[0]), out[2] = clip coefficient
__global__ void sumsq_final_kernel(const float* __restrict__ partials, int nparts, float* __restrict__ out,
                                   int accumulate, int finalize, float max_norm) {
  __shared__ float red[33];
  float s = 0.f;
  // fixed assignment of partials to threads + fixed-shape tree => deterministic
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partials[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    const float tot = (accumulate ? out[0] : 0.f) + s;
    out[0] = tot;
    if (finalize) {
      const float nrm = sqrtf(tot);
      out[1] = nrm;
      out[2] = (max_norm > 0.f && nrm > max_norm) ? max_norm / (nrm + 1e-6f) : 1.f;
    }
  }
}

__global__ void clip_finalize_kernel(float* __restrict__ out, float max_norm) {
  const float nrm = sqrtf(out[0]);
  out[1] = nrm;
  out[2] = (max_norm > 0.f && nrm > max_norm) ? max_norm / (nrm + 1e-6f) : 1.f;
}

__global__ void scale_kernel(float* __restrict__ x, long long n, const float* __restrict__ coef, float mul) {
  const float c = (coef ? *coef : 1.f) * mul;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    x[i] *= c;
}

__global__ void sgd_kernel(float* __restrict__ p, float* __restrict__ buf, const float* __restrict__ g,
                           __nv_bfloat16* __restrict__ p16, long long n, float lr, float momentum, float wd,
                           int nesterov) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float gg = g[i] + wd * p[i];
    if (buf) {
      const float b = momentum * buf[i] + gg;
      buf[i] = b;
      gg = nesterov ? gg + momentum * b : b;
    }
    const float pp = p[i] - lr * gg;
    p[i] = pp;
    if (p16) p16[i] = __float2bfloat16(pp);
  }
}

__global__ void lion_kernel(float* __restrict__ p, float* __restrict__ m, const float* __restrict__ g,
                            __nv_bfloat16* __restrict__ p16, long long n, float lr, float b1, float b2, float wd) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gg = g[i], mm = m[i];
    const float u = b1 * mm + (1.f - b1) * gg;
    const float sgn = (u > 0.f) - (u < 0.f);
    float pp = p[i];
    pp -= lr * (sgn + wd * pp);
    m[i] = b2 * mm + (1.f - b2) * gg;
    p[i] = pp;
    if (p16) p16[i] = __float2bfloat16(pp);
  }
}

static inline int nblocks(long long n, int per) {
  long long b = (n + per - 1) / per;
  return (int)(b < 1 ? 1 : (b > 148 * 8 ? 148 * 8 : b));
}

}  // namespace sx
using namespace sx;

extern "C" int sx_adamw_flat(float* p, float* m, float* v, const void* g, int g_bf16, void* p16, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, int step, float grad_scale,
                             const float* clip, cudaStream_t st) {
  if (n <= 0) return 0;
  AdamHyper h{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), grad_scale};
  const int nb = nblocks(n, 1024);
  if (g_bf16) adamw_flat_kernel<true><<<nb, 256, 0, st>>>(p, m, v, g, (__nv_bfloat16*)p16, n, h, clip);
  else adamw_flat_kernel<false><<<nb, 256, 0, st>>>(p, m, v, g, (__nv_bfloat16*)p16, n, h, clip);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Tensor-list AdamW: arrays of `count` device pointers / sizes held in HOST memory.
extern "C" int sx_adamw_multi(float** p, float** m, float** v, const void** g, int g_bf16, void** p16,
                              const long long* n, const float* wd, int count, float lr, float beta1, float beta2,
                              float eps, int step, float grad_scale, const float* clip, cudaStream_t st) {
  AdamHyper h{lr, beta1, beta2, eps, 0.f, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), grad_scale};
  for (int base = 0; base < count; base += MT_MAX) {
    MultiTensorTable tb;
    tb.count = count - base < MT_MAX ? count - base : MT_MAX;
    long long maxn = 0;
    for (int i = 0; i < tb.count; ++i) {
      tb.p[i] = p[base + i]; tb.m[i] = m[base + i]; tb.v[i] = v[base + i]; tb.g[i] = g[base + i];
      tb.p16[i] = p16 ? (__nv_bfloat16*)p16[base + i] : nullptr;
      tb.n[i] = n[base + i]; tb.wd[i] = wd[base + i];
      if (tb.n[i] > maxn) maxn = tb.n[i];
    }
    dim3 grid(nblocks(maxn, 2048) > 512 ? 512 : nblocks(maxn, 2048), tb.count);
    if (g_bf16) adamw_multi_kernel<true><<<grid, 256, 0, st>>>(tb, h, clip);
    else adamw_multi_kernel<false><<<grid, 256, 0, st>>>(tb, h, clip);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_sumsq_max_parts() { return 1024; }

// out: 3 floats {sum of squares, norm, clip coefficient}. partials: scratch of sx_sumsq_max_parts() floats.
extern "C" int sx_grad_sumsq(const void* g, int g_bf16, long long n, float* partials, float* out, int* nonfinite,
                             int accumulate, int finalize, float max_norm, cudaStream_t st) {
  int nb = nblocks(n, 4096);
  if (nb > sx_sumsq_max_parts()) nb = sx_sumsq_max_parts();
  if (g_bf16) sumsq_partial_kernel<true><<<nb, 256, 0, st>>>(g, n, partials, nonfinite);
  else sumsq_partial_kernel<false><<<nb, 256, 0, st>>>(g, n, partials, nonfinite);
  sumsq_final_kernel<<<1, 256, 0, st>>>(partials, nb, out, accumulate, finalize, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_clip_finalize(float* out, float max_norm, cudaStream_t st) {
  clip_finalize_kernel<<<1, 1, 0, st>>>(out, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_scale_f32(float* x, long long n, const float* coef, float mul, cudaStream_t st) {
  if (n <= 0) return 0;
  scale_kernel<<<nblocks(n, 1024), 256, 0, st>>>(x, n, coef, mul);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_sgd(float* p, float* buf, const float* g, void* p16, long long n, float lr, float momentum, float wd,
                      int nesterov, cudaStream_t st) {
  if (n <= 0) return 0;
  sgd_kernel<<<nblocks(n, 1024), 256, 0, st>>>(p, buf, g, (__nv_bfloat16*)p16, n, lr, momentum, wd, nesterov);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_lion(float* p, float* m, const float* g, void* p16, long long n, float lr, float b1, float b2,
                       float wd, cudaStream_t st) {
  if (n <= 0) return 0;
  lion_kernel<<<nblocks(n, 1024), 256, 0, st>>>(p, m, g, (__nv_bfloat16*)p16, n, lr, b1, b2, wd);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
