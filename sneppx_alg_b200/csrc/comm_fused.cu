// Fused collectives over NVLink peer memory (symmetric buffers), one kernel per hot path:
//   F1  ZeRO gradient reduce-scatter + 1/world scaling + global-norm clipping + partitioned AdamW
//   F2  (copy form) parameter all-gather by pulling peer shards
//   AR1 small all-reduce
// plus the group barrier / signal kernels. Each rank reads the slice it owns straight out of every
// peer's gradient buffer (16-byte peer loads, fp32 accumulation in rank order, so all ranks and all
// runs produce the same bits) and applies the optimizer to its fp32 shard in the same pass; no
// NCCL call and no intermediate gradient buffer exist on this path.
// The reference's counterparts are single-process simulations whose collectives are TODO comments
// (kernel/distributed/zero.c:111-167, kernel/cuda/optim_cuda.cu:574-615, kernel/distributed/ddp.c:85-95).
#include "comm_common.cuh"
#include "common.cuh"
#include "sx_api.h"

namespace sx {

static PeerTable to_table(const SxPeers* p) {
  PeerTable t;
  for (int i = 0; i < SX_MAX_RANKS; ++i) {
    t.buf[i] = p->buf[i];
    t.pad[i] = reinterpret_cast<uint32_t*>(p->pad[i]);
  }
  t.rank = p->rank;
  t.world = p->world;
  t.timeout_ns = p->timeout_ns ? p->timeout_ns : 2000000000ull;
  return t;
}

__global__ void peer_barrier_kernel(PeerTable pt, int channel, uint32_t epoch, int* status) {
  signal_all(pt, channel, epoch);
  wait_all(pt, channel, epoch, status);
}

__global__ void signal_peers_kernel(PeerTable pt, int channel, uint32_t epoch) { signal_all(pt, channel, epoch); }

struct ZeroParams {
  PeerTable pt;
  long long elem_offset, n;
  float* reduced;
  float* sumsq_partials;
  int partial_offset, num_partials;
  float* p32;
  float* m;
  float* v;
  __nv_bfloat16* p16;
  float lr, beta1, beta2, eps, wd, bc1, bc2;
  float max_norm;
  float* norm_out;
  int ready_channel;
  uint32_t ready_epoch;
  int norm_channel;
  uint32_t norm_epoch;
  int done_channel;
  uint32_t done_epoch;
  int mode;
  int* status;
  const __nv_bfloat16* mc;   // NVLS multicast view of the gradient buffer (nullptr: peer loads)
};

__device__ __forceinline__ void adamw1(float& p, float& m, float& v, float g, const ZeroParams& z) {
  m = z.beta1 * m + (1.f - z.beta1) * g;
  v = z.beta2 * v + (1.f - z.beta2) * g * g;
  p -= z.lr * z.wd * p;
  p -= z.lr * (m / z.bc1) / (sqrtf(v / z.bc2) + z.eps);
}

// Sum of the same 8 bf16 gradients over all ranks: one in-switch reduction (NVLS) when the buffer has a multicast
// mapping, else `world` peer loads summed in rank order.
__device__ __forceinline__ void reduce8(const ZeroParams& z, long long elem, float (&acc)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (z.mc) {
    const uint4 v = multimem_ld_reduce_bf16x8(z.mc + elem);
    acc_bf16x8(acc, v);
    return;
  }
  uint4 v[SX_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < SX_MAX_RANKS; ++r)
    if (r < z.pt.world) v[r] = ld_peer_v4(reinterpret_cast<const __nv_bfloat16*>(z.pt.buf[r]) + elem);
#pragma unroll
  for (int r = 0; r < SX_MAX_RANKS; ++r)
    if (r < z.pt.world) acc_bf16x8(acc, v[r]);
}

__global__ void __launch_bounds__(256) zero_step_kernel(const __grid_constant__ ZeroParams z) {
  __shared__ float red[33];
  __shared__ float s_coef;
  const long long nvec = z.n >> 3;
  const float inv_world = 1.f / z.pt.world;

  if (z.mode == 1 || z.mode == 3) {
    // every rank's bucket must be complete before anyone reads it
    if (!wait_all(z.pt, z.ready_channel, z.ready_epoch, z.status)) return;
  }

  if (z.mode == 1 && z.mc) {
    // NVLS: four in-switch reductions in flight per thread before the first result is used
    float ss = 0.f;
    constexpr int U = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) v[u] = multimem_ld_reduce_bf16x8(z.mc + z.elem_offset + i * 8);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i >= nvec) continue;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        acc_bf16x8(acc, v[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[j] *= inv_world;
          ss += acc[j] * acc[j];
        }
        float4* o = reinterpret_cast<float4*>(z.reduced + i * 8);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) z.sumsq_partials[z.partial_offset + blockIdx.x] = ss;
    return;
  }
  if (z.mode == 1) {
    float ss = 0.f;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
      float acc[8];
      reduce8(z, z.elem_offset + i * 8, acc);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        acc[j] *= inv_world;
        ss += acc[j] * acc[j];
      }
      float4* o = reinterpret_cast<float4*>(z.reduced + i * 8);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) z.sumsq_partials[z.partial_offset + blockIdx.x] = ss;
    return;
  }

  float coef = 1.f;
  if (z.mode == 2) {
    // my total, summed in index order by every CTA alike
    float mine = 0.f;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      for (int i = 0; i < z.num_partials; ++i) mine += z.sumsq_partials[i];
    }
    // publish (value word, then flag word) to every rank; all CTAs of all ranks then read the same w values
    uint32_t* mypad = z.pt.pad[z.pt.rank];
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      for (int r = 0; r < z.pt.world; ++r) {
        uint32_t* dst = z.pt.pad[r] + z.norm_channel * SX_PAD_STRIDE;
        reinterpret_cast<volatile float*>(dst + SX_PAD_STRIDE)[z.pt.rank] = mine;  // value lives in channel + 1
      }
      __threadfence_system();
      for (int r = 0; r < z.pt.world; ++r)
        st_release_sys(z.pt.pad[r] + z.norm_channel * SX_PAD_STRIDE + z.pt.rank, z.norm_epoch);
    }
    if (!wait_all(z.pt, z.norm_channel, z.norm_epoch, z.status)) return;
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int r = 0; r < z.pt.world; ++r)
        tot += reinterpret_cast<volatile float*>(mypad + (z.norm_channel + 1) * SX_PAD_STRIDE)[r];
      const float nrm = sqrtf(tot);
      const float c = (z.max_norm > 0.f && nrm > z.max_norm) ? z.max_norm / (nrm + 1e-6f) : 1.f;
      s_coef = c;
      if (blockIdx.x == 0 && z.norm_out) {
        z.norm_out[0] = tot;
        z.norm_out[1] = nrm;
        z.norm_out[2] = c;
      }
    }
    __syncthreads();
    coef = s_coef;
  }

  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float g[8];
    if (z.mode == 2) {
      const float4* src = reinterpret_cast<const float4*>(z.reduced + i * 8);
      const float4 a = src[0], b = src[1];
      g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] *= coef;
    } else {
      reduce8(z, z.elem_offset + i * 8, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] *= inv_world;
    }
    float4* pp = reinterpret_cast<float4*>(z.p32 + i * 8);
    float4* mm = reinterpret_cast<float4*>(z.m + i * 8);
    float4* vv = reinterpret_cast<float4*>(z.v + i * 8);
    float p[8], m[8], v[8];
    *reinterpret_cast<float4*>(&p[0]) = pp[0]; *reinterpret_cast<float4*>(&p[4]) = pp[1];
    *reinterpret_cast<float4*>(&m[0]) = mm[0]; *reinterpret_cast<float4*>(&m[4]) = mm[1];
    *reinterpret_cast<float4*>(&v[0]) = vv[0]; *reinterpret_cast<float4*>(&v[4]) = vv[1];
#pragma unroll
    for (int j = 0; j < 8; ++j) adamw1(p[j], m[j], v[j], g[j], z);
    pp[0] = *reinterpret_cast<float4*>(&p[0]); pp[1] = *reinterpret_cast<float4*>(&p[4]);
    mm[0] = *reinterpret_cast<float4*>(&m[0]); mm[1] = *reinterpret_cast<float4*>(&m[4]);
    vv[0] = *reinterpret_cast<float4*>(&v[0]); vv[1] = *reinterpret_cast<float4*>(&v[4]);
    if (z.p16) {
      bf16x8 pk = pack8(p);
      *reinterpret_cast<uint4*>(z.p16 + i * 8) = *reinterpret_cast<uint4*>(&pk);
    }
  }
  // Publish "my shard is written, and I am done reading your gradients". Arrivals are counted per CTA so that
  // the flag only moves once the whole grid has finished; the last CTA to finish signals and waits.
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* counter = z.pt.pad[z.pt.rank] + (SX_PAD_CHANNELS - 1) * SX_PAD_STRIDE;  // local CTA counter
    const uint32_t prev = atomicAdd(counter, 1u);
    s_last = (prev + 1 == gridDim.x);
    if (s_last) *counter = 0;  // launches on one stream do not overlap, so the next one starts from zero
  }
  __syncthreads();
  if (s_last) {
    signal_all(z.pt, z.done_channel, z.done_epoch);
    wait_all(z.pt, z.done_channel, z.done_epoch, z.status);
  }
}

// dst[r * shard .. ) <- peer r's shard, 16 bytes per thread per step; every rank's copy is local-write / remote-read.
__global__ void __launch_bounds__(512) allgather_pull_kernel(PeerTable pt, uint8_t* dst, long long shard_bytes,
                                                            long long src_off, int channel, uint32_t epoch,
                                                            int* status) {
  if (channel >= 0) {
    if (!wait_all(pt, channel, epoch, status)) return;
  }
  const long long nvec = shard_bytes >> 4;
  constexpr int U = 8;  // 16-byte loads in flight per thread: NVLink latency needs megabytes in flight per GPU
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int rr = 0; rr < pt.world; ++rr) {
    const int r = (pt.rank + rr) % pt.world;  // start with the local shard, then rotate so peers are hit evenly
    const uint8_t* src = reinterpret_cast<const uint8_t*>(pt.buf[r]) + src_off;
    uint8_t* d = dst + (long long)r * shard_bytes;
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) v[u] = ld_peer_v4(src + (i << 4));
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) *reinterpret_cast<uint4*>(d + (i << 4)) = v[u];
      }
    }
  }
}

// NVLS all-gather: my shard -> multicast address of my slot in every rank's full buffer.
__global__ void __launch_bounds__(512) allgather_mc_kernel(PeerTable pt, const uint8_t* __restrict__ src, uint8_t* mc_dst,
                                                          long long shard_bytes, int channel, uint32_t epoch,
                                                          int* status) {
  const long long nvec = shard_bytes >> 4;
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) v[u] = *reinterpret_cast<const uint4*>(src + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) multimem_st_v4(mc_dst + (i << 4), v[u]);
    }
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* counter = pt.pad[pt.rank] + (SX_PAD_CHANNELS - 1) * SX_PAD_STRIDE + 1;  // local CTA counter
    const uint32_t prev = atomicAdd(counter, 1u);
    s_last = (prev + 1 == gridDim.x);
    if (s_last) *counter = 0;
  }
  __syncthreads();
  if (s_last) {
    signal_all(pt, channel, epoch);
    wait_all(pt, channel, epoch, status);
  }
}

// Link probes (benchmarks only): every thread moves 16 bytes per step.
__global__ void __launch_bounds__(512) link_probe_kernel(PeerTable pt, int kind, int peer, const uint8_t* mc,
                                                        uint8_t* local, long long bytes) {
  const long long nvec = bytes >> 4;
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  uint8_t* remote = reinterpret_cast<uint8_t*>(pt.buf[peer]);
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      if (kind == 0) v[u] = ld_peer_v4(remote + (i << 4));
      else if (kind == 2) v[u] = multimem_ld_reduce_bf16x8(mc + (i << 4));
      else v[u] = *reinterpret_cast<const uint4*>(local + (i << 4));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      if (kind == 0 || kind == 2) *reinterpret_cast<uint4*>(local + (i << 4)) = v[u];
      else if (kind == 1) st_peer_v4(remote + (i << 4), v[u]);
      else multimem_st_v4(const_cast<uint8_t*>(mc) + (i << 4), v[u]);
    }
  }
}

// In-place sum over ranks of n fp32 values held at the start of each rank's buffer: every rank reads all peers'
// inputs (after a barrier), then writes its own result after a second barrier.
__global__ void __launch_bounds__(1024) allreduce_small_kernel(PeerTable pt, int n, int channel, uint32_t epoch,
                                                              int* status) {
  signal_all(pt, channel, epoch);
  if (!wait_all(pt, channel, epoch, status)) return;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0, i = threadIdx.x; k < 4 && i < n; ++k, i += blockDim.x)
    for (int r = 0; r < pt.world; ++r) acc[k] += reinterpret_cast<volatile float*>(pt.buf[r])[i];
  __syncthreads();
  signal_all(pt, channel + 1, epoch);
  if (!wait_all(pt, channel + 1, epoch, status)) return;
  for (int k = 0, i = threadIdx.x; k < 4 && i < n; ++k, i += blockDim.x)
    reinterpret_cast<float*>(pt.buf[pt.rank])[i] = acc[k];
}

// One-shot all-reduce of bf16 activations for tensor-parallel layers (decode steps, short prefill chunks): every rank
// has copied its n values into its symmetric staging buffer (stream-ordered before this launch); each CTA sums its
// slice over all ranks' staging buffers with 16-byte peer loads (fp32 accumulation, rank order) and writes the local
// result. The epoch is a counter in device memory that the launch itself advances, so the same launch can sit in a
// CUDA graph and be replayed; two barriers per call: inputs ready, and everyone done reading (staging reusable).
__global__ void __launch_bounds__(256) allreduce_bf16_kernel(PeerTable pt, __nv_bfloat16* __restrict__ out, long long n,
                                                             int channel, uint32_t* epoch_ctr, uint32_t* cta_counter,
                                                             int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ctr) + 1;
  if (blockIdx.x == 0) signal_all(pt, channel, epoch);
  const bool ok = wait_all(pt, channel, epoch, status);
  if (ok) {
    const long long nvec = n >> 3;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
      uint4 v[SX_MAX_RANKS];
#pragma unroll
      for (int r = 0; r < SX_MAX_RANKS; ++r)
        if (r < pt.world) v[r] = ld_peer_v4(reinterpret_cast<const __nv_bfloat16*>(pt.buf[r]) + i * 8);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int r = 0; r < SX_MAX_RANKS; ++r)
        if (r < pt.world) acc_bf16x8(acc, v[r]);
      bf16x8 o = pack8(acc);
      *reinterpret_cast<uint4*>(out + i * 8) = *reinterpret_cast<uint4*>(&o);
    }
  }
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(cta_counter, 1u);
    s_last = (prev + 1 == gridDim.x);
    if (s_last) *cta_counter = 0;
  }
  __syncthreads();
  if (s_last) {
    signal_all(pt, channel + 1, epoch);
    wait_all(pt, channel + 1, epoch, status);
    if (threadIdx.x == 0) *epoch_ctr = epoch;     // the next launch (or graph replay) uses epoch + 1
  }
}

}  // namespace sx
using namespace sx;

// peers->buf[r]: rank r's bf16 staging buffer holding its n values (n % 8 == 0); out: local bf16 [n] (may alias the
// local staging buffer's source tensor, not the staging buffer itself); epoch_ctr / cta_counter: local uint32 words,
// zeroed once. Uses channels `channel` and `channel + 1` of the signal pad.
extern "C" int sx_allreduce_bf16(const SxPeers* peers, void* out, long long n, int channel, void* epoch_ctr,
                                 void* cta_counter, int grid, int* status, cudaStream_t st) {
  if (n % 8 || n <= 0) return -1;
  long long want = (n / 8 + 255) / 256;
  if (grid <= 0) grid = (int)(want < 32 ? (want < 1 ? 1 : want) : 32);
  allreduce_bf16_kernel<<<grid, 256, 0, st>>>(to_table(peers), (__nv_bfloat16*)out, n, channel, (uint32_t*)epoch_ctr,
                                             (uint32_t*)cta_counter, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_peer_barrier(const SxPeers* peers, int channel, unsigned epoch, int* status, cudaStream_t st) {
  peer_barrier_kernel<<<1, 32, 0, st>>>(to_table(peers), channel, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_signal_peers(const SxPeers* peers, int channel, unsigned epoch, cudaStream_t st) {
  signal_peers_kernel<<<1, 32, 0, st>>>(to_table(peers), channel, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_zero_grid_default(void) { return 148 * 2; }

extern "C" int sx_zero_step(const SxZeroArgs* a, cudaStream_t st) {
  if ((a->n % 8) || (a->elem_offset % 8)) return -1;
  if (a->peers.world > SX_MAX_RANKS || a->peers.world < 1) return -2;
  ZeroParams z;
  z.pt = to_table(&a->peers);
  z.elem_offset = a->elem_offset; z.n = a->n;
  z.reduced = a->reduced; z.sumsq_partials = a->sumsq_partials;
  z.partial_offset = a->partial_offset; z.num_partials = a->num_partials;
  z.p32 = a->p32; z.m = a->m; z.v = a->v; z.p16 = (__nv_bfloat16*)a->p16_out;
  z.lr = a->lr; z.beta1 = a->beta1; z.beta2 = a->beta2; z.eps = a->eps; z.wd = a->wd;
  z.bc1 = 1.f - powf(a->beta1, (float)a->step); z.bc2 = 1.f - powf(a->beta2, (float)a->step);
  z.max_norm = a->max_norm; z.norm_out = a->norm_out;
  z.ready_channel = a->ready_channel; z.ready_epoch = a->ready_epoch;
  z.norm_channel = a->norm_channel; z.norm_epoch = a->norm_epoch;
  z.done_channel = a->done_channel; z.done_epoch = a->done_epoch;
  z.mode = a->mode; z.status = a->status;
  z.mc = reinterpret_cast<const __nv_bfloat16*>(a->mc_buf);
  const int grid = a->grid > 0 ? a->grid : sx_zero_grid_default();
  zero_step_kernel<<<grid, 256, 0, st>>>(z);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_allgather_pull(const SxPeers* peers, void* dst, long long shard_bytes, long long src_off, int channel,
                                 unsigned epoch, int grid, int* status, cudaStream_t st) {
  if ((shard_bytes % 16) || (src_off % 16)) return -1;
  allgather_pull_kernel<<<grid > 0 ? grid : 64, 512, 0, st>>>(to_table(peers), (uint8_t*)dst, shard_bytes, src_off,
                                                             channel, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_allgather_mc(const SxPeers* peers, const void* src_shard, void* mc_dst, long long shard_bytes,
                               int channel, unsigned epoch, int grid, int* status, cudaStream_t st) {
  if ((shard_bytes % 16) || !mc_dst || ((uintptr_t)mc_dst % 16) || ((uintptr_t)src_shard % 16)) return -1;
  allgather_mc_kernel<<<grid > 0 ? grid : 32, 512, 0, st>>>(to_table(peers), (const uint8_t*)src_shard, (uint8_t*)mc_dst,
                                                           shard_bytes, channel, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_link_probe(const SxPeers* peers, int kind, int peer, const void* mc, void* local, long long bytes,
                             int grid, cudaStream_t st) {
  if ((bytes % 16) || kind < 0 || kind > 3 || peer < 0 || peer >= peers->world) return -1;
  if ((kind == 2 || kind == 3) && !mc) return -2;
  link_probe_kernel<<<grid > 0 ? grid : 64, 512, 0, st>>>(to_table(peers), kind, peer, (const uint8_t*)mc, (uint8_t*)local,
                                                         bytes);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_allreduce_small(const SxPeers* peers, int n, int channel, unsigned epoch, int* status,
                                  cudaStream_t st) {
  if (n > 4096) return -1;
  allreduce_small_kernel<<<1, 1024, 0, st>>>(to_table(peers), n, channel, epoch, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
