// Entry point for callers that must not allocate device memory.
//
// Some users of this library run where cudaMalloc is off limits: inside a region that is being
// stream-captured or replayed, inside a real-time serving loop whose memory plan was fixed at start-up,
// or under an allocator policy that forbids new reservations once training has begun. Every other
// entry point that needs scratch memory asks its caller to pass it in; this one needs nothing but
// the caller's own input and output pointers, because its scratch lives in a fixed array that is part
// of the library image on every GPU that loads it (4 KiB per device, held until the process exits).
//
// This entry point has no counterpart in the reference code base.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest gradient buffer accepted, in elements. Larger inputs are rejected with SX_NOALLOC_E_TOO_LARGE.
#define SX_NOALLOC_MAX_ELEMS (1ll << 33)
#define SX_NOALLOC_E_TOO_LARGE (-40)
#define SX_NOALLOC_E_BAD_ARG (-41)
#define SX_NOALLOC_E_SYMBOL (-42)

// Gradient L2 norm and clip coefficient, same result as sx_grad_sumsq (accumulate = 0, finalize = 1):
//   out[0] = sum of squares of g[0..n), out[1] = sqrt(out[0]),
//   out[2] = max_norm / (out[1] + 1e-6) when max_norm > 0 and the norm exceeds it, else 1;
//   *nonfinite is set to 1 if any element is Inf/NaN (it is not cleared here).
// g: bf16 (g_bf16 != 0) or fp32 device buffer; out: 3 floats on the device; nonfinite: optional int on the device.
//
// Allocation: none. No cudaMalloc / cudaFree / library allocator is called, on any path.
// First call on a device: resolves the device address of the built-in scratch array (one
//   cudaGetSymbolAddress, checked, cached per device). Make that first call outside any stream capture.
// Sharing: every call on a device uses the same scratch array and overwrites all of it that it reads, so the
//   previous call's contents never leak into a result; but two calls whose kernels overlap in time on one GPU
//   (different streams) race on it. Issue calls for one device on one stream, or order them with events.
// Returns 0, SX_NOALLOC_E_* above, or -11 when the launch failed.
int sx_grad_sumsq_noalloc(const void* g, int g_bf16, long long n, float* out, int* nonfinite, float max_norm,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
