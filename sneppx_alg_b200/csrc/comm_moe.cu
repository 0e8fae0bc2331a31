// Expert-parallel routing plan and the combine half of the SER all-to-all (F6), over symmetric memory.
//   sx_ep_plan     counts per expert -> exchanged between ranks through peer stores -> every rank derives the same
//                  layout of every owner's expert-sorted buffer (segments padded to 128 rows, source ranks in rank
//                  order inside a segment) -> destination (rank, row) of each routed entry, tile -> expert table,
//                  cumulative per-tile arrival targets for the fused dispatch (gemm_tc.cu, COMM 3).
//   sx_ep_combine  y[t] = base[t] + sum_r w[t,r] * ys_owner[row]  read straight from the owners' output buffers with
//                  peer loads (the return all-to-all and the top-k weighted sum are one pass), optionally also
//                  dw[t,r] = <dy[t], ys_owner[row]> for the backward pass.
// The reference declares sneppx_cuda_expert_alltoall without a body (algorithms/ser/cuda/ser_cuda.cuh:83-93) and its
// C all-to-all is a local memcpy (kernel/distributed/expert_parallel.c:70-94).
#include "comm_common.cuh"
#include "common.cuh"
#include "sx_api.h"

namespace sx {

constexpr int EP_MAX_E = 256;

static PeerTable ep_table(const SxPeers* p) {
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

__global__ void ep_count_kernel(const int* __restrict__ idx, long long n, int* __restrict__ counts) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int e = idx[i];
    if (e >= 0) atomicAdd(&counts[e], 1);
  }
}

// pt.buf[r]: rank r's count matrix int32 [world][E]. One CTA.
__global__ void __launch_bounds__(256) ep_exchange_kernel(PeerTable pt, const int* __restrict__ counts, int E,
                                                          int channel, uint32_t epoch, int* __restrict__ e_base,
                                                          int* __restrict__ cursors, int* __restrict__ tile_group,
                                                          int* __restrict__ k_ranges, uint32_t* __restrict__ tile_cum,
                                                          uint32_t* __restrict__ tile_expected, int* __restrict__ total_rows,
                                                          int max_tiles, int* status) {
  __shared__ int s_total[EP_MAX_E];
  __shared__ int s_prefix[EP_MAX_E];
  __shared__ int s_off[EP_MAX_E + 1];
  const int w = pt.world, E_local = E / w;
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int r = 0; r < w; ++r) reinterpret_cast<volatile int*>(pt.buf[r])[pt.rank * E + e] = counts[e];
  __threadfence_system();
  __syncthreads();
  signal_all(pt, channel, epoch);
  if (!wait_all(pt, channel, epoch, status)) return;
  const volatile int* C = reinterpret_cast<const volatile int*>(pt.buf[pt.rank]);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, pre = 0;
    for (int r = 0; r < w; ++r) {
      const int c = C[r * E + e];
      if (r < pt.rank) pre += c;
      tot += c;
    }
    s_total[e] = tot;
    s_prefix[e] = pre;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // padded offsets restart at 0 on every owner
    for (int o = 0; o < w; ++o) {
      int off = 0;
      for (int el = 0; el < E_local; ++el) {
        const int e = o * E_local + el;
        s_off[e] = off;
        off += (s_total[e] + 127) / 128 * 128;
      }
      if (o == pt.rank) s_off[E] = off;  // rows used in my own buffer
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    e_base[e] = s_off[e] + s_prefix[e];
    cursors[e] = 0;
  }
  if (threadIdx.x == 0) *total_rows = s_off[E];
  // tables for the experts this rank owns
  for (int el = threadIdx.x; el < E_local; el += blockDim.x) {
    const int e = pt.rank * E_local + el;
    const int pad = (s_total[e] + 127) / 128 * 128;
    // rows past the end of the buffer are dropped by their senders (capacity), so the ranges stop there too
    k_ranges[2 * el] = min(s_off[e], max_tiles * 128);
    k_ranges[2 * el + 1] = min(s_off[e] + pad, max_tiles * 128);
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int row = t * 128;
    int g = -1, valid = 0;
    if (row < s_off[E]) {
      for (int el = 0; el < E_local; ++el) {
        const int e = pt.rank * E_local + el;
        const int pad = (s_total[e] + 127) / 128 * 128;
        if (row >= s_off[e] && row < s_off[e] + pad) {
          g = el;
          valid = min(128, max(0, s_total[e] - (row - s_off[e])));
          break;
        }
      }
    }
    tile_group[t] = g;
    const uint32_t cum = tile_cum[t] + (uint32_t)valid;
    tile_cum[t] = cum;
    tile_expected[t] = cum;
  }
}

__global__ void ep_assign_kernel(const int* __restrict__ idx, long long n, const int* __restrict__ e_base,
                                 int* __restrict__ cursors, int E_local, int max_rows, int* __restrict__ dest_rank,
                                 int* __restrict__ dest_row, int* __restrict__ dropped) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int e = idx[i];
    if (e < 0) {
      dest_rank[i] = -1;
      dest_row[i] = 0;
    } else {
      const int row = e_base[e] + atomicAdd(&cursors[e], 1);
      if (row >= max_rows) {  // past the owner's capacity: the entry is dropped (its gate weight gets no gradient)
        dest_rank[i] = -1;
        dest_row[i] = 0;
        atomicAdd(dropped, 1);
      } else {
        dest_rank[i] = e / E_local;
        dest_row[i] = row;
      }
    }
  }
}

// pt.buf[r]: rank r's expert-output buffer [rows, d] bf16. One warp per token.
__global__ void __launch_bounds__(256) ep_combine_kernel(PeerTable pt, const int* __restrict__ dest_rank,
                                                         const int* __restrict__ dest_row, const float* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ base,
                                                         const __nv_bfloat16* __restrict__ dy,
                                                         __nv_bfloat16* __restrict__ y, float* __restrict__ dw, int T, int d,
                                                         int k, int channel, uint32_t epoch, int done_channel,
                                                         uint32_t* cta_counter, int* status) {
  // every owner's outputs must be complete: each rank signals at the start of this kernel, i.e. after its own
  // expert GEMM in stream order
  if (blockIdx.x == 0) signal_all(pt, channel, epoch);
  const bool ok = wait_all(pt, channel, epoch, status);
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nw = (gridDim.x * blockDim.x) >> 5;
  if (ok) {
    for (int t = warp; t < T; t += nw) {
      float dots[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) dots[r] = 0.f;
      for (int c = lane * 8; c < d; c += 256) {
        float acc[8], g[8];
        if (base) unpack8(ld8(base + (long long)t * d + c), acc);
        else {
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        }
        if (dy) unpack8(ld8(dy + (long long)t * d + c), g);
        for (int r = 0; r < k; ++r) {
          const int dr = dest_rank[(long long)t * k + r];
          if (dr < 0) continue;
          const long long row = dest_row[(long long)t * k + r];
          const uint4 raw = ld_peer_v4(reinterpret_cast<const __nv_bfloat16*>(pt.buf[dr]) + row * d + c);
          float v[8];
          unpack8(*reinterpret_cast<const bf16x8*>(&raw), v);
          const float ww = w ? w[(long long)t * k + r] : 1.f;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[j] += ww * v[j];
            if (dy) dots[r] += g[j] * v[j];
          }
        }
        if (y) st8(y + (long long)t * d + c, pack8(acc));
      }
      if (dw) {
        for (int r = 0; r < k; ++r) {
          const float s = warp_sum(dots[r]);
          if (lane == 0) dw[(long long)t * k + r] = dest_rank[(long long)t * k + r] < 0 ? 0.f : s;
        }
      }
    }
  }
  // the owners may reuse their buffers once every rank has finished reading
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
    signal_all(pt, done_channel, epoch);
    wait_all(pt, done_channel, epoch, status);
  }
}

}  // namespace sx
using namespace sx;

// peers->buf[r]: rank r's int32 [world * E] count matrix. counts: int32 [E] scratch. Outputs (all int32, local):
// e_base [E], cursors [E], tile_group [max_tiles], k_ranges [2 * E/world], dest_rank / dest_row [n], total_rows [1];
// tile_cum (persistent uint32 [max_tiles], zeroed once) and tile_expected (uint32 [max_tiles]).
extern "C" int sx_ep_plan(const SxPeers* peers, const int* idx, long long n, int E, int* counts, int channel,
                          unsigned epoch, int* e_base, int* cursors, int* tile_group, int* k_ranges, void* tile_cum,
                          void* tile_expected, int* total_rows, int max_tiles, int* dest_rank, int* dest_row, int* dropped,
                          int* status,
                          cudaStream_t st) {
  if (E > EP_MAX_E || E % peers->world) return -1;
  cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  const int blocks = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  ep_count_kernel<<<blocks < 1 ? 1 : blocks, 256, 0, st>>>(idx, n, counts);
  ep_exchange_kernel<<<1, 256, 0, st>>>(ep_table(peers), counts, E, channel, epoch, e_base, cursors, tile_group, k_ranges,
                                        (uint32_t*)tile_cum, (uint32_t*)tile_expected, total_rows, max_tiles, status);
  ep_assign_kernel<<<blocks < 1 ? 1 : blocks, 256, 0, st>>>(idx, n, e_base, cursors, E / peers->world, max_tiles * 128, dest_rank,
                                                            dest_row, dropped);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ep_combine(const SxPeers* peers, const int* dest_rank, const int* dest_row, const float* w,
                             const void* base, const void* dy, void* y, float* dw, int T, int d, int k, int channel,
                             unsigned epoch, int done_channel, void* cta_counter, int* status, cudaStream_t st) {
  if (d % 8 || k > 8) return -1;
  ep_combine_kernel<<<148 * 2, 256, 0, st>>>(ep_table(peers), dest_rank, dest_row, w, (const __nv_bfloat16*)base,
                                             (const __nv_bfloat16*)dy, (__nv_bfloat16*)y, dw, T, d, k, channel, epoch,
                                             done_channel, (uint32_t*)cta_counter, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
