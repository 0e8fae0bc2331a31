// Q1: block-scaled quantisation. fp8 e4m3 with 1x128 (activation) and 128x128 (weight) fp32 scales, saturating
// conversion; INT4 symmetric group quantisation (group 128 along K, two values per byte, offset-8 nibbles); the
// matching dequantisers. Encode semantics follow the reference's saturating e4m3 codec
// (kernel/quantization/quantize_fp8.c) and its CUDA quantise kernels (kernel/quantization/quantize_cuda.cu:32-173),
// which had no block scales and no dequant-GEMM.
#include <cuda_fp8.h>
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr float E4M3_MAX = 448.f;

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// one warp per (row, 128-column block); lane handles 4 consecutive values
__global__ void quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scales, long long T, int K) {
  const int kb = K / 128;
  const long long nblk = T * kb;
  const int lane = threadIdx.x & 31;
  for (long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; w < nblk;
       w += ((long long)gridDim.x * blockDim.x) >> 5) {
    const long long t = w / kb;
    const int b = w % kb;
    const __nv_bfloat16* src = x + t * K + b * 128 + lane * 4;
    float v[4];
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = amax > 0.f ? amax / E4M3_MAX : 1.f;
    const float inv = 1.f / scale;
    uchar4 o;
    o.x = to_e4m3(v[0] * inv); o.y = to_e4m3(v[1] * inv); o.z = to_e4m3(v[2] * inv); o.w = to_e4m3(v[3] * inv);
    *reinterpret_cast<uchar4*>(q + t * K + b * 128 + lane * 4) = o;
    if (lane == 0) scales[t * kb + b] = scale;
  }
}

// one CTA (256 threads) per 128x128 block of w [N, K]
__global__ void __launch_bounds__(256) quant_fp8_128x128_kernel(const __nv_bfloat16* __restrict__ w,
                                                                uint8_t* __restrict__ q, float* __restrict__ scales,
                                                                int N, int K) {
  __shared__ float red[33];
  const int kb = (K + 127) / 128;
  const int bn = blockIdx.x / kb, bk = blockIdx.x % kb;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = bn * 128 + i / 128, c = bk * 128 + i % 128;
    if (r < N && c < K) amax = fmaxf(amax, fabsf(__bfloat162float(w[(long long)r * K + c])));
  }
  amax = block_max(amax, red);
  const float scale = amax > 0.f ? amax / E4M3_MAX : 1.f;
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = bn * 128 + i / 128, c = bk * 128 + i % 128;
    if (r < N && c < K) q[(long long)r * K + c] = to_e4m3(__bfloat162float(w[(long long)r * K + c]) * inv);
  }
  if (threadIdx.x == 0) scales[blockIdx.x] = scale;
}

// mode 0: 1x128 scales [rows, K/128]; mode 1: 128x128 scales [ceil(rows/128), ceil(K/128)]
__global__ void dequant_fp8_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                   __nv_bfloat16* __restrict__ out, long long rows, int K, int mode) {
  const long long n = rows * K;
  const int kb = (K + 127) / 128;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / K;
    const int c = i % K;
    const float s = mode == 0 ? scales[r * kb + c / 128] : scales[(r / 128) * kb + c / 128];
    out[i] = __float2bfloat16(from_e4m3(q[i]) * s);
  }
}

// INT4: one warp per (row, 128-column group); packed[r, c/2] = (q[c] + 8) | ((q[c+1] + 8) << 4)
__global__ void quant_int4_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ packed,
                                  float* __restrict__ scales, long long N, int K) {
  const int kb = K / 128;
  const long long nblk = N * kb;
  const int lane = threadIdx.x & 31;
  for (long long g = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; g < nblk;
       g += ((long long)gridDim.x * blockDim.x) >> 5) {
    const long long r = g / kb;
    const int b = g % kb;
    const __nv_bfloat16* src = w + r * K + b * 128 + lane * 4;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(src[j]);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = amax > 0.f ? amax / 7.f : 1.f;
    const float inv = 1.f / scale;
    int qv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) qv[j] = max(-8, min(7, __float2int_rn(v[j] * inv))) + 8;
    uchar2 o;
    o.x = (uint8_t)(qv[0] | (qv[1] << 4));
    o.y = (uint8_t)(qv[2] | (qv[3] << 4));
    *reinterpret_cast<uchar2*>(packed + r * (K / 2) + b * 64 + lane * 2) = o;
    if (lane == 0) scales[r * kb + b] = scale;
  }
}

__global__ void dequant_int4_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                    __nv_bfloat16* __restrict__ out, long long N, int K) {
  const long long n = N * (K / 2);
  const int kb = K / 128;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (K / 2);
    const int c = (i % (K / 2)) * 2;
    const float s = scales[r * kb + c / 128];
    const uint8_t b = packed[i];
    out[r * K + c] = __float2bfloat16(((int)(b & 15) - 8) * s);
    out[r * K + c + 1] = __float2bfloat16(((int)(b >> 4) - 8) * s);
  }
}

static inline int gridfor(long long n, int per) {
  long long b = (n + per - 1) / per;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace sx
using namespace sx;

extern "C" int sx_quant_fp8_1x128(const void* x, void* q, float* scales, long long T, int K, cudaStream_t st) {
  if (K % 128) return -1;
  quant_fp8_1x128_kernel<<<gridfor(T * (K / 128) * 32, 256), 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)q, scales, T, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
extern "C" int sx_quant_fp8_128x128(const void* w, void* q, float* scales, int N, int K, cudaStream_t st) {
  const int blocks = ((N + 127) / 128) * ((K + 127) / 128);
  quant_fp8_128x128_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)w, (uint8_t*)q, scales, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
extern "C" int sx_dequant_fp8(const void* q, const float* scales, void* out, long long rows, int K, int mode,
                              cudaStream_t st) {
  dequant_fp8_kernel<<<gridfor(rows * K, 256), 256, 0, st>>>((const uint8_t*)q, scales, (__nv_bfloat16*)out, rows, K, mode);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
extern "C" int sx_quant_int4(const void* w, void* packed, float* scales, long long N, int K, cudaStream_t st) {
  if (K % 128) return -1;
  quant_int4_kernel<<<gridfor(N * (K / 128) * 32, 256), 256, 0, st>>>((const __nv_bfloat16*)w, (uint8_t*)packed, scales, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
extern "C" int sx_dequant_int4(const void* packed, const float* scales, void* out, long long N, int K, cudaStream_t st) {
  if (K % 128) return -1;
  dequant_int4_kernel<<<gridfor(N * (K / 2), 256), 256, 0, st>>>((const uint8_t*)packed, scales, (__nv_bfloat16*)out, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
