// Device-side primitives for kernels that talk to peer GPUs over NVLink / NVSwitch through
// symmetric memory: system-scope release/acquire flags with BOUNDED waits, peer vector loads and
// stores, and NVLS multimem reductions. A wait that runs out writes ST_TIMEOUT_SIGNAL into the
// status word and returns false; callers then skip their remaining work and return normally.
//
// Flag protocol: every flag is a monotonically increasing 32-bit epoch; a consumer waits for
// "flag >= epoch", so flags never need resetting and a late reader cannot miss a signal.
// Pad layout (per rank, uint32 words): word [channel * SX_PAD_STRIDE + src_rank].
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define SX_MAX_RANKS 8
#define SX_PAD_STRIDE 16      // words per channel
#define SX_PAD_CHANNELS 64    // channels per pad
#define SX_PAD_WORDS (SX_PAD_STRIDE * SX_PAD_CHANNELS)

namespace sx {

struct PeerTable {
  void* buf[SX_MAX_RANKS];       // peer-mapped base of the symmetric data buffer on every rank
  uint32_t* pad[SX_MAX_RANKS];   // peer-mapped signal pad of every rank
  int rank, world;
  unsigned long long timeout_ns;  // bound of every flag wait in the kernel
};

__device__ __forceinline__ uint64_t comm_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait for *flag >= epoch at system scope (flag written by a peer GPU).
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns,
                                              int* status) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = comm_timer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
    if (((++spins) & 63u) == 0u) {
      if (comm_timer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, 4 /* ST_TIMEOUT_SIGNAL */);
        return false;
      }
      __nanosleep(64);
    }
  }
  return true;
}
// Same at device scope (flag written by another CTA of this GPU).
__device__ __forceinline__ bool wait_flag_gpu(const uint32_t* flag, uint32_t epoch, unsigned long long timeout_ns,
                                              int* status) {
  if ((int32_t)(ld_acquire_gpu(flag) - epoch) >= 0) return true;
  const uint64_t t0 = comm_timer_ns();
  uint32_t spins = 0;
  while ((int32_t)(ld_acquire_gpu(flag) - epoch) < 0) {
    if (((++spins) & 63u) == 0u) {
      if (comm_timer_ns() - t0 > timeout_ns) {
        if (status) atomicCAS(status, 0, 4);
        return false;
      }
      __nanosleep(32);
    }
  }
  return true;
}

// Every rank tells every rank "I reached `epoch` on `channel`". Called by one CTA; threads 0..world-1 send.
__device__ __forceinline__ void signal_all(const PeerTable& pt, int channel, uint32_t epoch) {
  if (threadIdx.x < pt.world) {
    __threadfence_system();
    st_release_sys(pt.pad[threadIdx.x] + channel * SX_PAD_STRIDE + pt.rank, epoch);
  }
}
// Wait until every rank has signalled `epoch` on `channel` of MY pad. Called by a whole CTA; result is CTA-uniform.
__device__ __forceinline__ bool wait_all(const PeerTable& pt, int channel, uint32_t epoch, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < pt.world) {
    if (!wait_flag_sys(pt.pad[pt.rank] + channel * SX_PAD_STRIDE + threadIdx.x, epoch, pt.timeout_ns, status)) s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  __syncthreads();  // every thread has read s_ok before a following wait_all may set it again
  return ok;
}

__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_peer_v4(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void acc_bf16x8(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// NVLS: one load that returns the sum over all ranks of 8 bf16 values (fp32 accumulation in the switch),
// and one store that lands on every rank. `mc` is an address inside the multicast mapping.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

}  // namespace sx
