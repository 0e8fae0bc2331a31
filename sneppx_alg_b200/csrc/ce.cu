// L1: fused softmax cross-entropy over one chunk of logits. One pass computes the row max and
// log-sum-exp online, a second pass overwrites the logits with their gradient
// (softmax - onehot) * scale, so the vocabulary-sized activation is read twice and written once
// and never exists in fp32. The vocab-chunked linear + CE driver on the Python side calls this
// between the logits GEMM and the two gradient GEMMs.
// Takes the place of the reference's softmax / cross-entropy backward kernels
// (kernel/cuda/autodiff_cuda.cu:519-608).
#include "common.cuh"
#include "sx_api.h"

namespace sx {

template <typename T>
__device__ __forceinline__ float ldf(const T* p, long long i);
template <>
__device__ __forceinline__ float ldf<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
__device__ __forceinline__ void stf(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// logits: [T, V] (row stride ld). loss[t] = lse - logit[target]; rows with target == ignore give 0.
// scale: device scalar (e.g. 1/num_valid_tokens) or null (1.0); write_grad: overwrite logits.
template <typename T>
__global__ void __launch_bounds__(512) ce_fwd_bwd_kernel(T* __restrict__ logits, const long long* __restrict__ target,
                                                         float* __restrict__ loss, float* __restrict__ lse_out,
                                                         int V, long long ld, long long ignore_index,
                                                         const float* __restrict__ scale, float scale_mul,
                                                         int write_grad) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  T* lr = logits + row * ld;
  const long long tgt = target[row];
  float mx = -INFINITY, sum = 0.f;
  if (sizeof(T) == 2 && (V % 8 == 0) && (ld % 8 == 0)) {
    const int nv = V >> 3;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float f[8];
      unpack8(ld8(reinterpret_cast<const __nv_bfloat16*>(lr) + i * 8), f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > mx) {
        sum *= __expf(mx - lm);
        mx = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += __expf(f[j] - mx);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = ldf(lr, i);
      if (x > mx) {
        sum *= __expf(mx - x);
        mx = x;
      }
      sum += __expf(x - mx);
    }
  }
  const float gmx = block_max(mx, red);
  sum = (mx == -INFINITY) ? 0.f : sum * __expf(mx - gmx);
  sum = block_sum(sum, red);
  const float lse = gmx + __logf(sum);
  const bool valid = (tgt != ignore_index) && tgt >= 0 && tgt < V;
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    loss[row] = valid ? lse - ldf(lr, tgt) : 0.f;
  }
  if (!write_grad) return;
  const float sc = valid ? (scale ? *scale : 1.f) * scale_mul : 0.f;
  if (sizeof(T) == 2 && (V % 8 == 0) && (ld % 8 == 0)) {
    const int nv = V >> 3;
    __nv_bfloat16* lb = reinterpret_cast<__nv_bfloat16*>(lr);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float f[8];
      unpack8(ld8(lb + i * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = __expf(f[j] - lse);
        if ((long long)(i * 8 + j) == tgt) g -= 1.f;
        f[j] = g * sc;
      }
      st8(lb + i * 8, pack8(f));
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float g = __expf(ldf(lr, i) - lse);
      if (i == tgt) g -= 1.f;
      stf(lr, i, g * sc);
    }
  }
}

__global__ void count_valid_kernel(const long long* __restrict__ target, long long n, long long ignore_index,
                                   float* __restrict__ inv_count) {
  __shared__ float red[33];
  float c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += (target[i] != ignore_index) ? 1.f : 0.f;
  c = block_sum(c, red);
  if (threadIdx.x == 0) inv_count[0] = c > 0.f ? 1.f / c : 0.f;
}

}  // namespace sx
using namespace sx;

extern "C" int sx_cross_entropy(void* logits, int logits_fp32, const long long* target, float* loss, float* lse,
                                long long T, int V, long long ld, long long ignore_index, const float* scale,
                                float scale_mul, int write_grad, cudaStream_t st) {
  if (T == 0) return 0;
  if (logits_fp32)
    ce_fwd_bwd_kernel<float><<<(unsigned)T, 512, 0, st>>>((float*)logits, target, loss, lse, V, ld, ignore_index,
                                                          scale, scale_mul, write_grad);
  else
    ce_fwd_bwd_kernel<__nv_bfloat16><<<(unsigned)T, 512, 0, st>>>((__nv_bfloat16*)logits, target, loss, lse, V, ld,
                                                                  ignore_index, scale, scale_mul, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_count_valid(const long long* target, long long n, long long ignore_index, float* inv_count,
                              cudaStream_t st) {
  count_valid_kernel<<<1, 1024, 0, st>>>(target, n, ignore_index, inv_count);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
