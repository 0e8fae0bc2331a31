// Debug-bounds support: index validation without traps. Index arrays that drive gathers / scatters (MoE slots,
// row -> token maps, paged-KV block tables and slot maps, loss targets, expert-dispatch destinations) are checked
// by a small kernel BEFORE the kernel that uses them runs; the first value outside [lo, hi) is recorded
// (site, position, value, limits) in a device record that the host reads with sx_debug_record_read. Nothing faults:
// the caller sees the record, skips the launch and raises. Outputs can be filled with a NaN pattern first
// (sx_debug_poison) so that an element a kernel failed to write shows up in the result.
// The reference's counterpart is a bounds-check macro that calls assert() on the device under SNEPPX_DEBUG
// (kernel/cuda/common.cuh:172-181) and a sanitizer script (scripts/run_sanitizers.sh:15-73).
#include <cuda_runtime.h>
#include <stdint.h>

namespace sx {

// [0] site (0: nothing recorded), [1] position in the array, [2] offending value, [3] lo, [4] hi
__device__ long long g_debug_record[5];

__global__ void debug_check_indices_kernel(const int* __restrict__ idx, long long n, long long lo, long long hi,
                                           int site, long long* rec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long v = idx[i];
    if (v < lo || v >= hi) {
      if (atomicCAS(reinterpret_cast<unsigned long long*>(rec), 0ull, (unsigned long long)site) == 0ull) {
        rec[1] = i;
        rec[2] = v;
        rec[3] = lo;
        rec[4] = hi;
      }
      return;
    }
  }
}

__global__ void debug_check_indices64_kernel(const long long* __restrict__ idx, long long n, long long lo, long long hi,
                                             long long also_ok, int site, long long* rec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long v = idx[i];
    if ((v < lo || v >= hi) && v != also_ok) {
      if (atomicCAS(reinterpret_cast<unsigned long long*>(rec), 0ull, (unsigned long long)site) == 0ull) {
        rec[1] = i;
        rec[2] = v;
        rec[3] = lo;
        rec[4] = hi;
      }
      return;
    }
  }
}

__global__ void debug_poison_kernel(uint32_t* __restrict__ p, long long words, uint32_t pattern) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < words; i += (long long)gridDim.x * blockDim.x)
    p[i] = pattern;
}

static long long* record_ptr() {
  long long* p = nullptr;
  return cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_debug_record) == cudaSuccess ? p : nullptr;
}

}  // namespace sx
using namespace sx;

// Every idx[i] must lie in [lo, hi); int32 values. `site` (> 0) names the caller in the record.
extern "C" int sx_debug_check_indices(const int* idx, long long n, long long lo, long long hi, int site,
                                      cudaStream_t st) {
  long long* rec = record_ptr();
  if (!rec || site <= 0) return -1;
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  debug_check_indices_kernel<<<blocks, 256, 0, st>>>(idx, n, lo, hi, site, rec);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// int64 values; `also_ok` is one extra accepted value (an ignore index).
extern "C" int sx_debug_check_indices64(const long long* idx, long long n, long long lo, long long hi, long long also_ok,
                                        int site, cudaStream_t st) {
  long long* rec = record_ptr();
  if (!rec || site <= 0) return -1;
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  debug_check_indices64_kernel<<<blocks, 256, 0, st>>>(idx, n, lo, hi, also_ok, site, rec);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Fill `bytes` (a multiple of 4) with a 32-bit pattern; 0x7FC07FC0 reads as NaN in bf16 pairs, 0x7FC00000 in fp32.
extern "C" int sx_debug_poison(void* p, long long bytes, unsigned pattern, cudaStream_t st) {
  if (bytes % 4 || (reinterpret_cast<uintptr_t>(p) & 3)) return -1;
  const long long words = bytes / 4;
  if (words == 0) return 0;
  const int blocks = (int)((words + 255) / 256 < 1184 ? (words + 255) / 256 : 1184);
  debug_poison_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<uint32_t*>(p), words, pattern);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// Synchronising read of the record into out[5]; optionally clears it.
extern "C" int sx_debug_record_read(long long* out5, int reset) {
  if (cudaMemcpyFromSymbol(out5, g_debug_record, sizeof(long long) * 5) != cudaSuccess) return -1;
  if (reset && out5[0] != 0) {
    long long zero[5] = {0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_debug_record, zero, sizeof(zero)) != cudaSuccess) return -2;
  }
  return 0;
}
