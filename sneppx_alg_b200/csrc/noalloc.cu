// Allocation-free gradient-norm entry point (see sx_noalloc.h for who needs it and why).
// Same two-stage reduction as sx_grad_sumsq in optim.cu: stage 1 writes one partial per CTA, stage 2 adds
// them in index order; only the home of the partials differs: a file-scope device array instead of a
// caller-supplied buffer.
#include "common.cuh"
#include "sx_noalloc.h"

namespace {

constexpr int kMaxParts = 1024;

// Scratch for the per-CTA partial sums. In host code this name is only a handle for the symbol; the device
// address is obtained once per device with cudaGetSymbolAddress below and passed to the kernels.
static __device__ __align__(256) float g_noalloc_partials[kMaxParts];

template <bool G_BF16>
__global__ void __launch_bounds__(256) na_sumsq_partial(const void* __restrict__ g, long long n,
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
  s = sx::block_sum(s, red);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;  // every slot that stage 2 reads is rewritten by this launch
  if (bad && nonfinite) atomicExch(nonfinite, 1);
}

__global__ void na_sumsq_final(const float* __restrict__ partials, int nparts, float* __restrict__ out,
                               float max_norm) {
  __shared__ float red[33];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partials[i];
  s = sx::block_sum(s, red);
  if (threadIdx.x == 0) {
    const float nrm = sqrtf(s);
    out[0] = s;
    out[1] = nrm;
    out[2] = (max_norm > 0.f && nrm > max_norm) ? max_norm / (nrm + 1e-6f) : 1.f;
  }
}

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (resolved on first use per device).
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SX_NOALLOC_E_SYMBOL;
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_partials) != cudaSuccess || !p)
      return SX_NOALLOC_E_SYMBOL;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int sx_grad_sumsq_noalloc(const void* g, int g_bf16, long long n, float* out, int* nonfinite,
                                     float max_norm, cudaStream_t st) {
  if (!g || !out || n <= 0) return SX_NOALLOC_E_BAD_ARG;
  if (n > SX_NOALLOC_MAX_ELEMS) return SX_NOALLOC_E_TOO_LARGE;
  float* partials = nullptr;
  const int rc = scratch_for_current_device(&partials);
  if (rc) return rc;
  long long nb = (n + 4095) / 4096;
  if (nb < 1) nb = 1;
  if (nb > 148 * 8) nb = 148 * 8;   // same grid rule as sx_grad_sumsq, so both paths add in the same order
  if (nb > kMaxParts) nb = kMaxParts;
  if (g_bf16) na_sumsq_partial<true><<<(int)nb, 256, 0, st>>>(g, n, partials, nonfinite);
  else na_sumsq_partial<false><<<(int)nb, 256, 0, st>>>(g, n, partials, nonfinite);
  na_sumsq_final<<<1, 256, 0, st>>>(partials, (int)nb, out, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
