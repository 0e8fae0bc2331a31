// NPE bytecode interpreter kernel: one thread block per input row runs the whole program with its registers in
// shared memory, so a compiled MLP-style program costs one launch instead of one per instruction.
//
// Reference: algorithms/npe/cuda/npe_cuda.cu:23-117 (interpreter over fp16 registers, grid (1, B), 256 threads). The
// instruction semantics live in npe_body.h, which the CPU oracle includes too. Matrix operands stay in program memory
// and are read with consecutive threads on consecutive columns; this is an interpreter for small programs, not a
// GEMM (large layers belong to the tcgen05 GEMM path through the host VM's FUSED_LINEAR).
#include <cuda_runtime.h>

#include "npe_body.h"
#include "sx_api.h"

namespace sx {

struct NpeBlockCtx {
  float* red;   // 33 floats of shared memory
  __device__ int tid() const { return (int)threadIdx.x; }
  __device__ int nthreads() const { return (int)blockDim.x; }
  __device__ void sync() const { __syncthreads(); }
  template <class F> __device__ float reduce(float v, F f, float identity) {
    for (int o = 16; o; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
      v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : identity;
      for (int o = 16; o; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
      if (threadIdx.x == 0) red[32] = v;
    }
    __syncthreads();
    v = red[32];
    __syncthreads();
    return v;
  }
  __device__ float sum(float v) { return reduce(v, [](float a, float b) { return a + b; }, 0.f); }
  __device__ float max(float v) { return reduce(v, [](float a, float b) { return fmaxf(a, b); }, -INFINITY); }
};

__global__ void __launch_bounds__(256) npe_interp_kernel(const SxNpeIns* prog, int n, const float* mem, const float* x, int in_w,
                                                         float* out, int out_w, long long rows, int maxw) {
  extern __shared__ float slots[];
  __shared__ float red[33];
  NpeBlockCtx ctx{red};
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    sx_npe_exec_row(prog, n, mem, x + row * in_w, in_w, out + row * out_w, slots, maxw, ctx);
    __syncthreads();
  }
}

}  // namespace sx

extern "C" {

// Host-side check of a program: widest register and output width; see sx_npe_plan for the codes.
int sx_npe_plan_program(const int* prog8, int n, long long mem_size, int in_w, int* maxw, int* out_w) {
  if (n < 0 || n > 4096 || in_w < 1) return -1;
  return sx_npe_plan((const SxNpeIns*)prog8, n, mem_size, in_w, maxw, out_w);
}

// prog_dev: the [n, 8] int32 instruction table on the device (same bytes as prog_host, which the planner reads).
int sx_npe_run(const int* prog_host, const int* prog_dev, int n, const float* mem, long long mem_size, const float* x, long long rows,
               int in_w, float* out, int out_w_expected, cudaStream_t st) {
  int maxw = 0, out_w = 0;
  if (rows < 1) return -1;
  const int rc = sx_npe_plan_program(prog_host, n, mem_size, in_w, &maxw, &out_w);
  if (rc != 0) return rc;
  if (out_w != out_w_expected) return -2;
  const size_t smem = (size_t)(SX_NPE_REGS + 1) * maxw * sizeof(float);
  if (smem > 200 * 1024) return -4;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(sx::npe_interp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -5;
  const long long cap = 148 * 8;
  sx::npe_interp_kernel<<<(int)(rows < cap ? rows : cap), 256, smem, st>>>((const SxNpeIns*)prog_dev, n, mem, x, in_w, out, out_w, rows, maxw);
  return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

}  // extern "C"
