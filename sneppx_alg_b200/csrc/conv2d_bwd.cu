// conv2d backward (input, weight and bias gradients) as direct kernels.
//
// Reference: kernel/cuda/autodiff_cuda.cu:620-740 (conv2d backward, one thread per output with serial loops). The
// forward convolution of this framework goes through cuDNN; these kernels give the backward pass a native path for
// the small vision models (ViT patch embedding, GAN / diffusion toy networks), where convolutions are far from the
// step's critical path. Not tensor-core code: one thread per dx element, one 256-thread block per dw / db element
// with a shuffle + shared-memory reduction. fp32 or bf16 inputs, fp32 gradients out.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "conv2d_bwd_body.h"
#include "sx_api.h"

namespace sx {

template <class T> struct LoadF;
template <> struct LoadF<float> { const float* p; __host__ __device__ float operator()(long long i) const { return p[i]; } };
template <> struct LoadF<__nv_bfloat16> { const __nv_bfloat16* p; __device__ float operator()(long long i) const { return __bfloat162float(p[i]); } };

__device__ __forceinline__ float block_sum_256(float v) {
  __shared__ float warp[8];
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) warp[threadIdx.x >> 5] = v;
  __syncthreads();
  v = threadIdx.x < 8 ? warp[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) for (int o = 4; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;   // valid in thread 0
}

template <class T>
__global__ void conv2d_dx_kernel(SxConvDims d, const T* dy, const T* w, float* dx, long long total) {
  LoadF<T> ldy{dy}, lw{w};
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ww = (int)(i % d.W), h = (int)((i / d.W) % d.H), c = (int)((i / ((long long)d.W * d.H)) % d.C);
    const int n = (int)(i / ((long long)d.W * d.H * d.C));
    dx[i] = sx_conv2d_dx_at(d, ldy, lw, n, c, h, ww);
  }
}

template <class T>
__global__ void __launch_bounds__(256) conv2d_dw_kernel(SxConvDims d, const T* dy, const T* x, float* dw, int count) {
  LoadF<T> ldy{dy}, lx{x};
  for (int e = blockIdx.x; e < count; e += gridDim.x) {          // uniform per block: every thread reaches the barrier
    const int s = e % d.S, r = (e / d.S) % d.R, c = (e / (d.S * d.R)) % d.C, k = e / (d.S * d.R * d.C);
    const float v = block_sum_256(sx_conv2d_dw_partial(d, ldy, lx, k, c, r, s, threadIdx.x, 256));
    if (threadIdx.x == 0) dw[e] = v;
    __syncthreads();
  }
}

template <class T>
__global__ void __launch_bounds__(256) conv2d_db_kernel(SxConvDims d, const T* dy, float* db) {
  LoadF<T> ldy{dy};
  for (int k = blockIdx.x; k < d.K; k += gridDim.x) {
    const float v = block_sum_256(sx_conv2d_db_partial(d, ldy, k, threadIdx.x, 256));
    if (threadIdx.x == 0) db[k] = v;
    __syncthreads();
  }
}

template <class T>
int conv2d_bwd_launch(const SxConvDims& d, const void* x, const void* w, const void* dy, float* dx, float* dw, float* db, cudaStream_t st) {
  const long long nx = (long long)d.N * d.C * d.H * d.W;
  const int nw = d.K * d.C * d.R * d.S, cap = 148 * 16;
  if (dx) {
    const long long blocks = (nx + 255) / 256;
    conv2d_dx_kernel<T><<<(int)(blocks < cap ? blocks : cap), 256, 0, st>>>(d, (const T*)dy, (const T*)w, dx, nx);
  }
  if (dw) conv2d_dw_kernel<T><<<nw < cap ? nw : cap, 256, 0, st>>>(d, (const T*)dy, (const T*)x, dw, nw);
  if (db) conv2d_db_kernel<T><<<d.K < cap ? d.K : cap, 256, 0, st>>>(d, (const T*)dy, db);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace sx

extern "C" int sx_conv2d_bwd(const void* x, const void* w, const void* dy, float* dx, float* dw, float* db, int N, int C, int H,
                             int W, int K, int R, int S, int stride, int pad, int is_bf16, cudaStream_t st) {
  if (N < 1 || C < 1 || H < 1 || W < 1 || K < 1 || R < 1 || S < 1 || stride < 1 || pad < 0) return -1;
  if (H + 2 * pad < R || W + 2 * pad < S) return -1;
  if ((long long)K * C * R * S > (1LL << 30)) return -1;
  SxConvDims d{N, C, H, W, K, R, S, (H + 2 * pad - R) / stride + 1, (W + 2 * pad - S) / stride + 1, stride, pad};
  if ((dw && !x) || (dx && !w) || !dy) return -1;
  return is_bf16 ? sx::conv2d_bwd_launch<__nv_bfloat16>(d, x, w, dy, dx, dw, db, st) : sx::conv2d_bwd_launch<float>(d, x, w, dy, dx, dw, db, st);
}
