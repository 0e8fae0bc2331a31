// G1/G2: persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[b] = act(alpha * A[b] x B[b]^T + bias + beta * C[b])        (fp32 accumulation in TMEM)
//
// A is M x K, B is N x K (both "K-major", i.e. a torch Linear weight is a valid B as is); either
// operand may instead be stored transposed ("MN-major": [K, M] or [K, N] row-major), which covers
// dgrad (dX = dY x W) and wgrad (dW = dY^T x X) without any transposing copy.
// One kernel also serves the grouped (per-expert) GEMMs of the SER MoE layer: a per-M-tile table
// selects which B matrix a row block multiplies (forward / dgrad), and a per-batch reduction range
// restricts K to one expert's token segment (wgrad).
//
// Structure (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
// epilogue (TMEM -> registers -> global). CTA tile 128 x BN x 64, UMMA 128 x BN x 16, smem ring of
// STAGES tiles, two TMEM accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
// Takes the place of the reference's mma.sync / SIMT GEMMs (kernel/cuda/tensor_cuda.cu:28-285) and
// its cuBLAS backward calls (kernel/cuda/autodiff_cuda.cu:28-171).
#include <stdlib.h>
#include "tc_common.cuh"
#include "comm_common.cuh"
#include "common.cuh"
#include "tmap.h"
#include "sx_api.h"

namespace sx {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

// Collective fused into the GEMM (template parameter COMM):
//   COMM == 1  all-gather -> GEMM (F3 for activations, F2 for ZeRO-3 weights). The gathered operand (A rows or B rows)
//              is split in `world` chunks of chunk_rows rows; rank r's chunk lives at the same offset of rank r's copy of
//              the symmetric full-size buffer. The first n_copy CTAs pull remote chunks over NVLink in sub-chunks and
//              publish a device-scope flag per sub-chunk; the other CTAs run the GEMM with tiles ordered so that the
//              local chunk comes first, and their TMA producer waits for the flag of the sub-chunk a tile reads.
//   COMM == 2  GEMM -> reduce-scatter (F4). Output rows are split in `world` chunks; a tile that belongs to rank c is
//              written (bf16) into slot `rank` of c's symmetric staging buffer and counted on c's per-row-block counter
//              (system-scope release add). After its own tiles each CTA reduces row blocks of the local chunk in rank
//              order as soon as their counters are complete. Tiles are ordered remote chunks first, local chunk last.
// Every wait is bounded (pt.timeout_ns) and reports ST_TIMEOUT_SIGNAL through the status word.
struct CommParams {
  PeerTable pt;
  uint8_t* full;        // COMM 1: local full operand buffer (== pt.buf[rank])
  uint32_t* flags;      // COMM 1: local flags [world * subs_per_chunk]
  uint32_t epoch;
  int n_copy;           // COMM 1: CTAs that copy
  int gather_b;         // COMM 1: 0 = A rows are gathered, 1 = B rows
  int chunk_rows;       // rows per rank chunk (multiple of sub_rows)
  int sub_rows;         // COMM 1: rows per flag (multiple of 128 for A, of BN for B)
  long long row_bytes;  // COMM 1: bytes per row of the gathered operand
  int sig_channel, done_channel;
  int counter_word;     // COMM 2: first word of the row-block counters inside the signal pad
  uint32_t rs_expected; // COMM 2: counter value at which a row block of this call is complete
  void* rs_out;         // COMM 2: [chunk_rows, N] local result
  const void* rs_residual;  // COMM 2: optional [chunk_rows, N] added to the result
  long long rs_ldd;
  uint32_t* cta_counter;    // local word used to find the last CTA of the grid
  // COMM 3 (F5: expert all-to-all dispatch -> grouped GEMM). pt.buf[r] is rank r's expert-sorted row buffer
  // [rows, d]; the first n_copy CTAs push this rank's routed rows (optionally scaled) straight into the owners'
  // buffers and bump the owner's per-tile arrival counter; GEMM CTAs wait until a tile's counter reaches
  // tile_expected[tile] before reading it.
  const __nv_bfloat16* ep_x;     // [T, d] local tokens
  const int* ep_dest_rank;       // [T*k]  (-1: dropped)
  const int* ep_dest_row;        // [T*k]
  const float* ep_row_scale;     // optional [T*k]
  int ep_entries, ep_k, ep_d;
  uint32_t* ep_arrive[SX_MAX_RANKS];   // peer-mapped arrival counters, one word per 128-row tile
  const uint32_t* ep_tile_expected;    // local [m_blks] cumulative expected arrivals
};

struct GemmKernelParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  void* D;
  const void* C;
  const float* bias;
  const int* tile_group;  // grouped: per m-block index of the B batch (-1: skip)
  const int* k_ranges;    // per batch [k_begin, k_end)
  int* status;
  long long ldd, ldc, strideD, strideC;
  int M, N, K, batch;
  int a_batched, b_batched;
  int out_fp32, c_fp32, act;
  float alpha, beta;
  int m_blks, n_blks;
  CommParams cm;
};

template <int BN, int COMM = 0>
struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // GEMM -> reduce-scatter stages its bf16 output tile in shared memory (BM x BN x 2 bytes) so that rows leave for
  // the owner's staging buffer as whole 2*BN-byte runs; it pays for that with one pipeline stage.
  static constexpr int OUT_BYTES = COMM == 2 ? BM * BN * 2 : 0;
  static constexpr int STAGES = (BN == 256) ? (COMM == 2 ? 3 : 4) : (BN == 128 ? (COMM == 2 ? 5 : 6) : 8);
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int OFF_OUT = STAGES * STAGE_BYTES;
  static constexpr int OFF_BAR = OFF_OUT + OUT_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int t, int m_blks, int n_blks, int& b, int& m_blk, int& n_blk) {
  const int per_batch = m_blks * n_blks;
  b = t / per_batch;
  int r = t - b * per_batch;
  constexpr int GM = 8;
  const int group_sz = GM * n_blks;
  const int g = r / group_sz;
  const int first_m = g * GM;
  const int gsz = min(GM, m_blks - first_m);
  const int rr = r - g * group_sz;
  m_blk = first_m + rr % gsz;
  n_blk = rr / gsz;
}

template <int BN, bool A_MN, bool B_MN, int COMM>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tc_kernel(const __grid_constant__ GemmKernelParams p) {
  using Cfg = GemmCfg<BN, COMM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::OFF_BAR);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + Cfg::STAGES;       // [STAGES]
  uint64_t* tfull_bar = bars + 2 * Cfg::STAGES;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 4);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
  }
  const bool is_copy_cta = (COMM == 1 || COMM == 3) && ((int)blockIdx.x < p.cm.n_copy);
  if (warp == 1 && !is_copy_cta) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = is_copy_cta ? 0u : *tmem_slot;

  const int total_tiles = p.batch * p.m_blks * p.n_blks;
  // CTAs that run GEMM tiles: all of them, minus the copy CTAs of the all-gather form
  const int cta0 = (COMM == 1 || COMM == 3) ? p.cm.n_copy : 0;
  const int tile_first = (int)blockIdx.x - cta0;
  const int tile_step = (int)gridDim.x - cta0;
  // tile rotation so that every rank starts on rows it already has (COMM 1) / ends on rows it owns (COMM 2)
  int rot_m = 0, rot_n = 0;
  if (COMM == 1) {
    if (p.cm.gather_b) rot_n = p.cm.pt.rank * (p.cm.chunk_rows / BN);
    else rot_m = p.cm.pt.rank * (p.cm.chunk_rows / BM);
  } else if (COMM == 2) {
    rot_m = ((p.cm.pt.rank + 1) % p.cm.pt.world) * (p.cm.chunk_rows / BM);
  }

  if (is_copy_cta && COMM == 3) {
    // ------------------------------------------------------------ expert dispatch CTAs (push rows to their owners)
    const PeerTable& pt = p.cm.pt;
    __shared__ int s_ok3;
    // the owners clear their row buffers before this launch; tell everyone mine is ready, wait for theirs
    if (blockIdx.x == 0) signal_all(pt, p.cm.sig_channel, p.cm.epoch);
    const bool ready = wait_all(pt, p.cm.sig_channel, p.cm.epoch, p.status);
    (void)s_ok3;
    if (ready) {
      // A warp moves two rows at a time (all loads of both rows in flight before the first remote store) and makes its
      // rows visible in groups of 16: one system-scope fence, then one arrival count per row. A fence per row would
      // serialise the warp on the NVLink round trip (measured: 14 us per row, 7 ms per dispatch).
      const int d = p.cm.ep_d;
      const int nw = p.cm.n_copy * (GEMM_THREADS / 32);
      const int w0 = blockIdx.x * (GEMM_THREADS / 32) + warp;
      const int nvec = d / 256 + ((d % 256) ? 1 : 0);      // 16-byte vectors per lane per row (<= 8 handled unrolled)
      int pend_rank = -1, pend_tile = 0;                     // lane i holds the i-th pending (rank, tile) of the group
      int n_pend = 0;
      auto flush = [&]() {
        __threadfence_system();
        __syncwarp();
        if (lane < n_pend && pend_rank >= 0) red_release_sys_add(p.cm.ep_arrive[pend_rank] + pend_tile, 1u);
        n_pend = 0;
        pend_rank = -1;
      };
      for (int e0 = w0; e0 < p.cm.ep_entries; e0 += 2 * nw) {
        int dr[2], row[2];
        float sc[2];
        const __nv_bfloat16* src[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int e = e0 + u * nw;
          dr[u] = e < p.cm.ep_entries ? p.cm.ep_dest_rank[e] : -1;
          row[u] = dr[u] >= 0 ? p.cm.ep_dest_row[e] : 0;
          sc[u] = (dr[u] >= 0 && p.cm.ep_row_scale) ? p.cm.ep_row_scale[e] : 1.f;
          src[u] = p.cm.ep_x + (long long)((e < p.cm.ep_entries ? e : 0) / p.cm.ep_k) * d;
        }
        if (nvec <= 8) {
          bf16x8 v[2][8];
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int c = lane * 8 + i * 256;
              if (dr[u] >= 0 && c < d) v[u][i] = ld8(src[u] + c);
            }
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            if (dr[u] < 0) continue;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pt.buf[dr[u]]) + (long long)row[u] * d;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int c = lane * 8 + i * 256;
              if (c < d) {
                bf16x8 o = v[u][i];
                if (p.cm.ep_row_scale) {
                  float f[8];
                  unpack8(o, f);
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] *= sc[u];
                  o = pack8(f);
                }
                st_peer_v4(dst + c, *reinterpret_cast<uint4*>(&o));
              }
            }
          }
        } else {
          for (int u = 0; u < 2; ++u) {
            if (dr[u] < 0) continue;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(pt.buf[dr[u]]) + (long long)row[u] * d;
            for (int c = lane * 8; c < d; c += 256) {
              bf16x8 o = ld8(src[u] + c);
              if (p.cm.ep_row_scale) {
                float f[8];
                unpack8(o, f);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] *= sc[u];
                o = pack8(f);
              }
              st_peer_v4(dst + c, *reinterpret_cast<uint4*>(&o));
            }
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (dr[u] >= 0) {
            if (lane == n_pend) { pend_rank = dr[u]; pend_tile = row[u] >> 7; }
            ++n_pend;
          }
        }
        if (n_pend >= 16) flush();
      }
      flush();
    }
  } else if (is_copy_cta) {
    // ------------------------------------------------------------ all-gather copy CTAs
    const PeerTable& pt = p.cm.pt;
    __shared__ int s_ok;
    if (blockIdx.x == 0) signal_all(pt, p.cm.sig_channel, p.cm.epoch);  // my chunk is complete (stream order)
    const int subs = p.cm.chunk_rows / p.cm.sub_rows;
    const long long sub_bytes = (long long)p.cm.sub_rows * p.cm.row_bytes;
    bool ok = true;
    int copy_uses = 0;  // pieces issued so far by this CTA (gives ring slot and mbarrier parity)
    // Work items are (source rank, sub-block) pairs in the order the MMA CTAs consume them (nearest rank first), dealt
    // round-robin to the copy CTAs: every copy CTA has work from the start, also when a chunk has fewer sub-blocks
    // than there are copy CTAs (8 ranks x 1024 rows: 4 to 8 sub-blocks per rank).
    const int items = (pt.world - 1) * subs;
    unsigned seen = 0;  // ranks whose "chunk complete" signal this CTA has already observed
    for (int it = blockIdx.x; it < items && ok; it += p.cm.n_copy) {
      const int r = (pt.rank + 1 + it / subs) % pt.world;
      const int sub = it % subs;
      if (!((seen >> r) & 1u)) {
        if (threadIdx.x == 0)
          s_ok = wait_flag_sys(pt.pad[pt.rank] + p.cm.sig_channel * SX_PAD_STRIDE + r, p.cm.epoch, pt.timeout_ns, p.status);
        __syncthreads();
        ok = s_ok != 0;
        __syncthreads();
        if (!ok) break;
        seen |= 1u << r;
      }
      // One thread drives bulk copies peer -> shared -> local through a ring of 32 KB pieces in the (otherwise
      // unused) tile staging area, NBUF pieces in flight per CTA, so that a handful of CTAs keep NVLink full.
      constexpr int PIECE = 32768, NBUF = 4;
      {
        const long long off = ((long long)r * p.cm.chunk_rows + (long long)sub * p.cm.sub_rows) * p.cm.row_bytes;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(pt.buf[r]) + off;
        uint8_t* dst = p.cm.full + off;
        if (threadIdx.x == 0) {
          const int npieces = (int)((sub_bytes + PIECE - 1) / PIECE);
          int issued = 0, done = 0;
          bool good = true;
          while (done < npieces && good) {
            while (issued < npieces && issued - done < NBUF) {
              const int bidx = copy_uses % NBUF;
              const long long o = (long long)issued * PIECE;
              const uint32_t bytes = (uint32_t)min((long long)PIECE, sub_bytes - o);
              mbar_expect_tx(&full_bar[bidx], bytes);
              asm volatile(
                  "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                      smem_u32(smem + bidx * PIECE)),
                  "l"(src + o), "r"(bytes), "r"(smem_u32(&full_bar[bidx]))
                  : "memory");
              ++issued;
              ++copy_uses;
            }
            const int use = copy_uses - (issued - done);     // global index of the piece being retired
            const int bidx = use % NBUF;
            if (!mbar_wait(&full_bar[bidx], (use / NBUF) & 1, s_abort, p.status, ST_TIMEOUT_SIGNAL)) { good = false; break; }
            const long long o = (long long)done * PIECE;
            const uint32_t bytes = (uint32_t)min((long long)PIECE, sub_bytes - o);
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + o),
                         "r"(smem_u32(smem + bidx * PIECE)), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            ++done;
          }
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          if (good) st_release_gpu(&p.cm.flags[r * subs + sub], p.cm.epoch);
          s_ok = good ? 1 : 0;
        }
        __syncthreads();
        ok = s_ok != 0;
        __syncthreads();
      }
    }
  } else

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = tile_first; t < total_tiles && ok; t += tile_step) {
        int b, m_blk, n_blk;
        tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        if (COMM == 1 || COMM == 2) { m_blk = (m_blk + rot_m) % p.m_blks; n_blk = (n_blk + rot_n) % p.n_blks; }
        int bsel = b;
        if (p.tile_group) {
          bsel = p.tile_group[m_blk];
          if (bsel < 0) continue;
        }
        int k0 = 0, k1 = p.K;
        if (p.k_ranges) {
          k0 = p.k_ranges[2 * b];
          k1 = p.k_ranges[2 * b + 1];
        }
        const int ab = p.a_batched ? b : 0;
        const int bb = p.b_batched ? bsel : 0;
        const int num_kb = (k1 - k0 + BK - 1) / BK;
        if (COMM == 1) {
          const int row0 = p.cm.gather_b ? n_blk * BN : m_blk * BM;
          const int src = row0 / p.cm.chunk_rows;
          if (src != p.cm.pt.rank) {
            const int subs = p.cm.chunk_rows / p.cm.sub_rows;
            const int sub = (row0 - src * p.cm.chunk_rows) / p.cm.sub_rows;
            if (!wait_flag_gpu(&p.cm.flags[src * subs + sub], p.cm.epoch, p.cm.pt.timeout_ns, p.status)) {
              *s_abort = 1;
              ok = false;
              break;
            }
            // rows were written by ordinary stores of the copy CTAs; order them before this thread's TMA reads
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        if (COMM == 3) {
          if (!wait_flag_sys(p.cm.ep_arrive[p.cm.pt.rank] + m_blk, p.cm.ep_tile_expected[m_blk], p.cm.pt.timeout_ns,
                             p.status)) {
            *s_abort = 1;
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          const int kc = k0 + kb * BK;
          if (A_MN) tma_load_4d(sa, &p.tmA, &full_bar[stage], 0, kc, m_blk * (BM / 64), ab);
          else      tma_load_3d(sa, &p.tmA, &full_bar[stage], kc, m_blk * BM, ab);
          if (B_MN) tma_load_4d(sb, &p.tmB, &full_bar[stage], 0, kc, n_blk * (BN / 64), bb);
          else      tma_load_3d(sb, &p.tmB, &full_bar[stage], kc, n_blk * BN, bb);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = tile_first; t < total_tiles && ok; t += tile_step) {
        int b, m_blk, n_blk;
        tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        if (COMM == 1 || COMM == 2) { m_blk = (m_blk + rot_m) % p.m_blks; n_blk = (n_blk + rot_n) % p.n_blks; }
        if (p.tile_group && p.tile_group[m_blk] < 0) continue;
        int k0 = 0, k1 = p.K;
        if (p.k_ranges) {
          k0 = p.k_ranges[2 * b];
          k1 = p.k_ranges[2 * b + 1];
        }
        const int num_kb = (k1 - k0 + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (num_kb == 0) {
          // empty reduction range: nothing was accumulated; the epilogue treats it as zeros.
        }
        umma_commit(&tfull_bar[acc]);
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps, 128 rows)
    const int q = warp & 3;  // TMEM lane quadrant this warp may access
    int it = 0;
    bool ok = true;
    for (int t = tile_first; t < total_tiles && ok; t += tile_step) {
      int b, m_blk, n_blk;
      tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        if (COMM == 1 || COMM == 2) { m_blk = (m_blk + rot_m) % p.m_blks; n_blk = (n_blk + rot_n) % p.n_blks; }
      if (p.tile_group && p.tile_group[m_blk] < 0) continue;
      bool empty_k = false;
      if (p.k_ranges) empty_k = (p.k_ranges[2 * b + 1] <= p.k_ranges[2 * b]);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], acc_phase, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
      void* Dptr = p.D;
      int rs_owner = 0, rs_rb = 0;
      if (COMM == 2) {
        rs_owner = (m_blk * BM) / p.cm.chunk_rows;
        rs_rb = (m_blk * BM - rs_owner * p.cm.chunk_rows) / BM;
        Dptr = p.cm.pt.buf[rs_owner];   // owner's staging buffer, slot `rank`
        drow = ((long long)p.cm.pt.rank * p.cm.chunk_rows + (row - rs_owner * p.cm.chunk_rows)) * (long long)p.N;
      }
      const long long crow = (long long)b * p.strideC + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n_blk * BN + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = empty_k ? 0.f : __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || col0 + j < p.N) v[j] += p.bias[col0 + j];
        }
        if (p.beta != 0.f && p.C) {
          if (p.c_fp32) {
            const float* cp = reinterpret_cast<const float*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * cp[j];
          } else {
            const __nv_bfloat16* cp = reinterpret_cast<const __nv_bfloat16*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * __bfloat162float(cp[j]);
          }
        }
        if (p.act == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        } else if (p.act == 2) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
        } else if (p.act == 3) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        if (COMM == 2) {
          // this lane's 64 bytes of the row go to the warp's slab: 16-byte chunk index XOR row keeps both the writes
          // here (same chunk index, 32 rows) and the row-wise reads below free of bank conflicts
          uint8_t* slab = smem + Cfg::OFF_OUT + q * (32 * BN * 2) + lane * (BN * 2);
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(v[j], v[j + 1]);
            o.y = pack_bf16x2(v[j + 2], v[j + 3]);
            o.z = pack_bf16x2(v[j + 4], v[j + 5]);
            o.w = pack_bf16x2(v[j + 6], v[j + 7]);
            const int ci = c * 4 + (j >> 3);
            *reinterpret_cast<uint4*>(slab + (((ci ^ lane) & (BN / 8 - 1)) << 4)) = o;
          }
        } else if (p.out_fp32) {
          float* dp = reinterpret_cast<float*>(Dptr) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = v[j];
          }
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(Dptr) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16x2(v[j], v[j + 1]);
              o.y = pack_bf16x2(v[j + 2], v[j + 3]);
              o.z = pack_bf16x2(v[j + 4], v[j + 5]);
              o.w = pack_bf16x2(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(dp + j) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      if (COMM == 2) {
        // write the slab out row by row: lane l carries 16-byte chunk l (and l + 32 for BN = 256) of the row, so each
        // store instruction is one contiguous 512-byte run of the owner's staging buffer
        __syncwarp();
        const uint8_t* slab0 = smem + Cfg::OFF_OUT + q * (32 * BN * 2);
        const int row_base = m_blk * BM + q * 32;
        for (int rr = 0; rr < 32; ++rr) {
          const int grow = row_base + rr;
          if (grow >= p.M) break;
          __nv_bfloat16* drp = reinterpret_cast<__nv_bfloat16*>(Dptr) +
                               ((long long)p.cm.pt.rank * p.cm.chunk_rows + (grow - rs_owner * p.cm.chunk_rows)) * (long long)p.N +
                               n_blk * BN;
#pragma unroll
          for (int h = 0; h < BN / 256 + (BN % 256 ? 1 : 0); ++h) {
            const int ci = lane + h * 32;
            if (ci < BN / 8 && n_blk * BN + ci * 8 < p.N) {
              const uint4 o = *reinterpret_cast<const uint4*>(slab0 + rr * (BN * 2) + (((ci ^ rr) & (BN / 8 - 1)) << 4));
              st_peer_v4(drp + ci * 8, o);
            }
          }
        }
        __threadfence_system();   // partial tile visible to its owner before the count moves
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);
        if (COMM == 2) red_release_sys_add(p.cm.pt.pad[rs_owner] + p.cm.counter_word + rs_rb, 1u);
      }
      ++it;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);  // let copies in flight land before freeing
  if (warp == 1 && !is_copy_cta) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }

  if (COMM == 2) {
    // ---------------------------------------------------------- reduce the row blocks this rank owns
    const PeerTable& pt = p.cm.pt;
    __shared__ int s_ok2;
    const int blks = p.cm.chunk_rows / BM;
    const int units = blks * p.n_blks;
    const uint32_t expected = p.cm.rs_expected;  // cumulative arrivals per row block, tracked by the host per call site
    const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(pt.buf[pt.rank]);
    for (int u = tile_first; u < units; u += tile_step) {
      const int rb = u / p.n_blks, nb = u % p.n_blks;
      if (threadIdx.x == 0)
        s_ok2 = wait_flag_sys(pt.pad[pt.rank] + p.cm.counter_word + rb, expected, pt.timeout_ns, p.status);
      __syncthreads();
      const bool okk = s_ok2 != 0;
      __syncthreads();
      if (!okk) break;
      constexpr int VPR = BN / 8;  // 16-byte vectors per row of the strip
      for (int idx = threadIdx.x; idx < BM * VPR; idx += GEMM_THREADS) {
        const int rr = idx / VPR, col = nb * BN + (idx % VPR) * 8;
        if (col >= p.N) continue;
        const int lrow = rb * BM + rr;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < pt.world; ++r)
          acc_bf16x8(acc, ld_peer_v4(stage + ((long long)r * p.cm.chunk_rows + lrow) * p.N + col));
        if (p.cm.rs_residual) {
          float e[8];
          unpack8(ld8(reinterpret_cast<const __nv_bfloat16*>(p.cm.rs_residual) + (long long)lrow * p.cm.rs_ldd + col), e);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += e[j];
        }
        st8(reinterpret_cast<__nv_bfloat16*>(p.cm.rs_out) + (long long)lrow * p.cm.rs_ldd + col, pack8(acc));
      }
    }
  }
  if (COMM != 0) {
    // Last CTA of the grid tells the peers that this rank no longer reads their memory / has consumed its staging
    // buffer, and waits for the same from everyone, so the buffers may be reused once the kernel has returned.
    __shared__ int s_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t prev = atomicAdd(p.cm.cta_counter, 1u);
      s_last = (prev + 1 == gridDim.x);
      if (s_last) *p.cm.cta_counter = 0;
    }
    __syncthreads();
    if (s_last) {
      signal_all(p.cm.pt, p.cm.done_channel, p.cm.epoch);
      wait_all(p.cm.pt, p.cm.done_channel, p.cm.epoch, p.status);
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int COMM = 0>
static int launch_cfg(const GemmKernelParams& kp, int grid, cudaStream_t st) {
  using Cfg = GemmCfg<BN, COMM>;
  static bool attr_set = false;
  auto kern = gemm_tc_kernel<BN, A_MN, B_MN, COMM>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return -10;
    attr_set = true;
  }
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(kp);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static int make_operand_map(CUtensorMap* tm, const void* ptr, int mn, int K, long long ld, int batched, int batch,
                            long long stride, bool mn_major, int tile_mn) {
  if (mn_major) {
    if (mn % 64 != 0) return -20;
    uint64_t dims[4] = {64, (uint64_t)K, (uint64_t)(mn / 64), (uint64_t)(batched ? batch : 1)};
    uint64_t strides[3] = {(uint64_t)ld * 2, 128, (uint64_t)(batched ? stride : (long long)K * ld) * 2};
    uint32_t box[4] = {64, (uint32_t)BK, (uint32_t)(tile_mn / 64), 1};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptr, dims, strides, box);
  } else {
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)mn, (uint64_t)(batched ? batch : 1)};
    uint64_t strides[2] = {(uint64_t)ld * 2, (uint64_t)(batched ? stride : (long long)mn * ld) * 2};
    uint32_t box[3] = {(uint32_t)BK, (uint32_t)tile_mn, 1};
    return make_tmap(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ptr, dims, strides, box);
  }
}


// ================================================================================================
// G1 on a CTA pair: the same GEMM with `cta_group::2`. A cluster of two CTAs (two SMs) owns one 256 x 256 output
// tile: each CTA stages its own 128 rows of A and its own 128 rows of B per k-block (32 KB instead of the 48 KB a
// single CTA needs for 128 x 256), the even CTA's MMA thread issues 256 x 256 x 16 instructions that read both
// CTAs' shared memory, and each CTA's TMEM receives the accumulator rows of its A half. Per SM this halves the
// B-operand shared-memory traffic and leaves room for six pipeline stages.
// Protocol (barrier arrays live at the same shared-memory offsets in both CTAs):
//   full[s]   even CTA only: its producer arms 64 KB, the TMA loads of BOTH CTAs complete on it
//   empty[s]  both CTAs: released by the even CTA's tcgen05.commit, multicast to the pair
//   tfull[a]  both CTAs: accumulator a complete, multicast commit
//   tempty[a] even CTA only, 8 arrivals: the four epilogue warps of each CTA arrive on it (the odd CTA remotely)
// Dense, non-grouped, non-fused calls only; everything else stays on gemm_tc_kernel.
// Pair tile 256 x BN2 (BN2 = 256, or 128 when the wider tile would leave the last wave of pairs mostly idle).
template <int BN2>
struct G2Cfg {
  static constexpr int STAGES = BN2 == 256 ? 6 : 8;
  static constexpr int A_BYTES = 128 * BK * 2;          // 16 KB
  static constexpr int B_BYTES = (BN2 / 2) * BK * 2;    // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the even CTA's copy

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma2_load_3d(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1,
                                             int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma2_load_4d(void* dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void umma2_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// Arrives (once the MMAs issued so far have executed) on the barrier at this offset in BOTH CTAs of the pair.
__device__ __forceinline__ void umma2_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_even_cta(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}

template <int BN2, bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm2_kernel(const __grid_constant__ GemmKernelParams p) {
  constexpr int G2_STAGES = G2Cfg<BN2>::STAGES;
  constexpr int G2_A_BYTES = G2Cfg<BN2>::A_BYTES;
  constexpr int G2_STAGE_BYTES = G2Cfg<BN2>::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G2_STAGES * G2_STAGE_BYTES);
  uint64_t* full_bar = bars;                     // [STAGES]
  uint64_t* empty_bar = bars + G2_STAGES;        // [STAGES]
  uint64_t* tfull_bar = bars + 2 * G2_STAGES;    // [2]
  uint64_t* tempty_bar = tfull_bar + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0: issues the MMAs, owns full[] / tempty[]
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull_bar[i], 1);
      mbar_init(&tempty_bar[i], 8);
    }
    *s_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&p.tmA);
    tma_prefetch_desc(&p.tmB);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before any remote arrive or TMA completion
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // p.m_blks counts 256-row pair tiles, p.n_blks BN2-column tiles
  const int total_tiles = p.batch * p.m_blks * p.n_blks;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cluster_id; t < total_tiles; t += n_clusters) {
        int b, m_blk, n_blk;
        tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
        const int ab = p.a_batched ? b : 0, bb = p.b_batched ? b : 0;
        const int num_kb = (p.K + BK - 1) / BK;
        const int arow = m_blk * 256 + (int)rank * 128, brow = n_blk * BN2 + (int)rank * (BN2 / 2);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, s_abort, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          uint8_t* sa = smem + stage * G2_STAGE_BYTES;
          uint8_t* sb = sa + G2_A_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * G2_STAGE_BYTES);
          const uint32_t fb = smem_u32(&full_bar[stage]) & PEER_MASK;
          const int kc = kb * BK;
          if (A_MN) tma2_load_4d(sa, &p.tmA, fb, 0, kc, arow / 64, ab);
          else      tma2_load_3d(sa, &p.tmA, fb, kc, arow, ab);
          if (B_MN) tma2_load_4d(sb, &p.tmB, fb, 0, kc, brow / 64, bb);
          else      tma2_load_3d(sb, &p.tmB, fb, kc, brow, bb);
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(256, BN2, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = cluster_id; t < total_tiles && ok; t += n_clusters) {
        const int num_kb = (p.K + BK - 1) / BK;
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, s_abort, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, s_abort, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * G2_STAGE_BYTES);
          const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                        : umma_desc_sw128(sb + k * 32, 16, 1024);
            umma2_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma2_commit_pair(&empty_bar[stage]);
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma2_commit_pair(&tfull_bar[acc]);
        ++it;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps per CTA, this CTA's 128 rows)
    const int q = warp & 3;
    int it = 0;
    for (int t = cluster_id; t < total_tiles; t += n_clusters) {
      int b, m_blk, n_blk;
      tile_coords(t, p.m_blks, p.n_blks, b, m_blk, n_blk);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait_warp(&tfull_bar[acc], acc_phase, s_abort, p.status, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m_blk * 256 + (int)rank * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long drow = (long long)b * p.strideD + (long long)row * p.ldd;
      const long long crow = (long long)b * p.strideC + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN2 / 32; ++c) {
        const int col0 = n_blk * BN2 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN2 + c * 32 + (static_cast<uint32_t>(q * 32) << 16), r);
        tmem_ld_wait();
        if (!row_ok) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        const bool full = (col0 + 32 <= p.N);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (full || col0 + j < p.N) v[j] += p.bias[col0 + j];
        }
        if (p.beta != 0.f && p.C) {
          if (p.c_fp32) {
            const float* cp = reinterpret_cast<const float*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * cp[j];
          } else {
            const __nv_bfloat16* cp = reinterpret_cast<const __nv_bfloat16*>(p.C) + crow + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (full || col0 + j < p.N) v[j] += p.beta * __bfloat162float(cp[j]);
          }
        }
        if (p.act == 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh(v[j]);
        } else if (p.act == 2) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu(v[j]);
        } else if (p.act == 3) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.f);
        }
        if (p.out_fp32) {
          float* dp = reinterpret_cast<float*>(p.D) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(dp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = v[j];
          }
        } else {
          __nv_bfloat16* dp = reinterpret_cast<__nv_bfloat16*>(p.D) + drow + col0;
          if (full && ((reinterpret_cast<uintptr_t>(dp) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16x2(v[j], v[j + 1]);
              o.y = pack_bf16x2(v[j + 2], v[j + 3]);
              o.z = pack_bf16x2(v[j + 4], v[j + 5]);
              o.w = pack_bf16x2(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(dp + j) = o;
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) dp[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_even_cta(&tempty_bar[acc]);
      ++it;
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (*s_abort) bounded_delay_ns(2000000);  // let copies in flight land before freeing
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its peer may still read its memory or signal it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

static int g2_max_clusters(int sms) {
  // the largest number of 2-CTA clusters of this kernel family that can be co-resident (74 on a 148-SM part)
  return sms / 2;
}

template <int BN2, bool A_MN, bool B_MN>
static int launch_cfg2(const GemmKernelParams& kp, int sms, cudaStream_t st) {
  static bool attr_set = false;
  static int max_clusters = 0;
  auto kern = gemm2_kernel<BN2, A_MN, B_MN>;
  constexpr int SMEM = G2Cfg<BN2>::SMEM_BYTES;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -10;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms & ~1, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters <= 0) {
      cudaGetLastError();
      max_clusters = g2_max_clusters(sms);
    }
    attr_set = true;
  }
  const long long tiles = (long long)kp.batch * kp.m_blks * kp.n_blks;
  int clusters = (int)(tiles < max_clusters ? tiles : max_clusters);
  if (clusters > sms / 2) clusters = sms / 2;
  kern<<<2 * clusters, GEMM_THREADS, SMEM, st>>>(kp);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

template <int BN2>
static int launch_cfg2_any(const GemmKernelParams& kp, int am, int bm, int sms, cudaStream_t st) {
  if (!am && !bm) return launch_cfg2<BN2, false, false>(kp, sms, st);
  if (!am && bm) return launch_cfg2<BN2, false, true>(kp, sms, st);
  if (am && !bm) return launch_cfg2<BN2, true, false>(kp, sms, st);
  return launch_cfg2<BN2, true, true>(kp, sms, st);
}

}  // namespace sx

extern "C" int sx_gemm_skinny_ok(const SxGemmArgs* a);
extern "C" int sx_gemm_skinny(const SxGemmArgs* a, cudaStream_t st);

static int gemm_launch(const SxGemmArgs* a, const SxGemmCommArgs* cm, cudaStream_t st) {
  using namespace sx;
  if (a->M <= 0 || a->N <= 0 || a->batch <= 0) return 0;
  // decode-sized products stream the weight on the cluster split-K kernel (gemm_skinny.cu)
  if (!cm && sx_gemm_skinny_ok(a)) return sx_gemm_skinny(a, st);
  if ((a->lda % 8) || (a->ldb % 8) || (reinterpret_cast<uintptr_t>(a->A) & 15) ||
      (reinterpret_cast<uintptr_t>(a->B) & 15))
    return -1;
  if (a->K % 8) return -2;
  GemmKernelParams kp;
  int BN = (a->N > 128 || a->force_bn == 256) && a->force_bn != 128 ? 256 : 128;
  if (cm && cm->mode == 2 && (cm->sub_rows % 256) != 0) BN = 128;
  const int a_batched = a->strideA != 0 && a->batch > 1;
  const int b_batched = (a->strideB != 0 && a->batch > 1) || a->tile_group != nullptr;
  const int b_nbatch = a->tile_group ? a->num_groups : a->batch;
  // Reduction length seen by the tensor maps: total K rows/cols of the operand storage.
  const int Kfull = a->k_ranges ? a->k_total : a->K;
  // CTA-pair kernel for plain dense products that fill at least one 256 x 256 pair tile.
  static int use_pair = -1;
  if (use_pair < 0) {
    const char* e = getenv("SX_GEMM_2CTA");  // set to 0 to force the single-CTA kernel
    use_pair = e ? atoi(e) : 1;
  }
  if (use_pair && !cm && !a->tile_group && !a->k_ranges && a->M >= 256 && a->N >= 256 && a->force_bn == 0 &&
      a->sm_limit == 0 && (!a->a_mn || a->M % 64 == 0) && (!a->b_mn || a->N % 64 == 0)) {
    const int bb2 = a->strideB != 0 && a->batch > 1;
    int dev2 = 0, sms2 = 148;
    cudaGetDevice(&dev2);
    cudaDeviceGetAttribute(&sms2, cudaDevAttrMultiProcessorCount, dev2);
    // Tile width: 256. The 256 x 128 pair tile measured 0.75 of a 256 x 256 tile's time (not the ~0.53 that would make
    // it pay off against wave quantisation), so it is only taken on request (force_bn == 128 through SX_GEMM_PAIR_BN).
    static int pair_bn = 0;
    if (pair_bn == 0) {
      const char* e = getenv("SX_GEMM_PAIR_BN");
      pair_bn = (e && atoi(e) == 128) ? 128 : 256;
    }
    const int bn2 = pair_bn;
    int rc2 = make_operand_map(&kp.tmA, a->A, a->M, a->K, a->lda, a_batched, a->batch, a->strideA, a->a_mn != 0, 128);
    if (rc2) return rc2;
    rc2 = make_operand_map(&kp.tmB, a->B, a->N, a->K, a->ldb, bb2, a->batch, a->strideB, a->b_mn != 0, bn2 / 2);
    if (rc2) return rc2;
    kp.D = a->D; kp.C = a->C; kp.bias = a->bias; kp.tile_group = nullptr; kp.k_ranges = nullptr; kp.status = a->status;
    kp.ldd = a->ldd; kp.ldc = a->ldc; kp.strideD = a->strideD; kp.strideC = a->strideC;
    kp.M = a->M; kp.N = a->N; kp.K = a->K; kp.batch = a->batch;
    kp.a_batched = a_batched; kp.b_batched = bb2;
    kp.out_fp32 = a->out_fp32; kp.c_fp32 = a->c_fp32; kp.act = a->act; kp.alpha = a->alpha; kp.beta = a->beta;
    kp.m_blks = (a->M + 255) / 256; kp.n_blks = (a->N + bn2 - 1) / bn2;
    const int am2 = a->a_mn != 0, bm2 = a->b_mn != 0;
    return bn2 == 256 ? launch_cfg2_any<256>(kp, am2, bm2, sms2, st) : launch_cfg2_any<128>(kp, am2, bm2, sms2, st);
  }
  int rc = make_operand_map(&kp.tmA, a->A, a->M, Kfull, a->lda, a_batched, a->batch, a->strideA, a->a_mn != 0, BM);
  if (rc) return rc;
  rc = make_operand_map(&kp.tmB, a->B, a->N, Kfull, a->ldb, b_batched, b_nbatch, a->strideB, a->b_mn != 0, BN);
  if (rc) return rc;
  kp.D = a->D;
  kp.C = a->C;
  kp.bias = a->bias;
  kp.tile_group = a->tile_group;
  kp.k_ranges = a->k_ranges;
  kp.status = a->status;
  kp.ldd = a->ldd;
  kp.ldc = a->ldc;
  kp.strideD = a->strideD;
  kp.strideC = a->strideC;
  kp.M = a->M;
  kp.N = a->N;
  kp.K = a->K;
  kp.batch = a->batch;
  kp.a_batched = a_batched;
  kp.b_batched = b_batched;
  kp.out_fp32 = a->out_fp32;
  kp.c_fp32 = a->c_fp32;
  kp.act = a->act;
  kp.alpha = a->alpha;
  kp.beta = a->beta;
  kp.m_blks = (a->M + BM - 1) / BM;
  kp.n_blks = (a->N + BN - 1) / BN;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  static int cached_sms[16] = {0};
  if (dev < 16 && cached_sms[dev] == 0) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cached_sms[dev] = sms;
  }
  if (dev < 16) sms = cached_sms[dev];
  if (a->sm_limit > 0 && a->sm_limit < sms) sms = a->sm_limit;
  const long long tiles = (long long)kp.batch * kp.m_blks * kp.n_blks;
  int grid = (int)(tiles < sms ? tiles : sms);
  const int am = a->a_mn != 0, bm = a->b_mn != 0;
  if (cm) {
    if (am || a->batch != 1 || a->k_ranges) return -30;
    if ((cm->mode == 4) != (a->tile_group != nullptr)) return -30;
    CommParams& c = kp.cm;
    for (int i = 0; i < SX_MAX_RANKS; ++i) {
      c.pt.buf[i] = cm->peers.buf[i];
      c.pt.pad[i] = reinterpret_cast<uint32_t*>(cm->peers.pad[i]);
    }
    c.pt.rank = cm->peers.rank;
    c.pt.world = cm->peers.world;
    c.pt.timeout_ns = cm->peers.timeout_ns ? cm->peers.timeout_ns : 2000000000ull;
    c.flags = reinterpret_cast<uint32_t*>(cm->flags);
    c.epoch = cm->epoch;
    c.chunk_rows = cm->chunk_rows;
    c.sub_rows = cm->sub_rows;
    c.sig_channel = cm->sig_channel;
    c.done_channel = cm->done_channel;
    c.counter_word = cm->counter_word;
    c.rs_expected = cm->rs_expected;
    c.rs_out = cm->rs_out;
    c.rs_residual = cm->rs_residual;
    c.rs_ldd = cm->rs_ldd;
    c.cta_counter = reinterpret_cast<uint32_t*>(cm->cta_counter);
    c.n_copy = 0;
    c.gather_b = 0;
    if (cm->mode == 1 || cm->mode == 2) {
      c.gather_b = cm->mode == 2;
      const int rows_total = c.gather_b ? a->N : a->M;
      const int tile_rows = c.gather_b ? BN : BM;
      if (cm->chunk_rows * cm->peers.world != rows_total || (cm->chunk_rows % cm->sub_rows) ||
          (cm->sub_rows % tile_rows) || (a->K % 8))
        return -31;
      c.full = reinterpret_cast<uint8_t*>(cm->peers.buf[cm->peers.rank]);
      c.row_bytes = (long long)(c.gather_b ? a->ldb : a->lda) * 2;
      c.n_copy = cm->n_copy > 0 ? cm->n_copy : 8;
      if (cm->peers.world == 1) c.n_copy = 0;
      if (grid + c.n_copy > sms) grid = sms - c.n_copy;
      grid += c.n_copy;  // every CTA must be resident at once: copy CTAs feed the GEMM CTAs of the same launch
      if (!bm) return BN == 256 ? launch_cfg<256, false, false, 1>(kp, grid, st) : launch_cfg<128, false, false, 1>(kp, grid, st);
      return BN == 256 ? launch_cfg<256, false, true, 1>(kp, grid, st) : launch_cfg<128, false, true, 1>(kp, grid, st);
    } else if (cm->mode == 3) {
      if (cm->chunk_rows * cm->peers.world != a->M || (cm->chunk_rows % BM) || a->out_fp32 || (a->N % 8)) return -32;
      if (!bm) return BN == 256 ? launch_cfg<256, false, false, 2>(kp, grid, st) : launch_cfg<128, false, false, 2>(kp, grid, st);
      return BN == 256 ? launch_cfg<256, false, true, 2>(kp, grid, st) : launch_cfg<128, false, true, 2>(kp, grid, st);
    }
    else if (cm->mode == 4) {
      if (cm->ep_d % 8) return -34;
      c.ep_x = reinterpret_cast<const __nv_bfloat16*>(cm->ep_x);
      c.ep_dest_rank = cm->ep_dest_rank;
      c.ep_dest_row = cm->ep_dest_row;
      c.ep_row_scale = cm->ep_row_scale;
      c.ep_entries = cm->ep_entries;
      c.ep_k = cm->ep_k;
      c.ep_d = cm->ep_d;
      for (int i = 0; i < SX_MAX_RANKS; ++i) c.ep_arrive[i] = reinterpret_cast<uint32_t*>(cm->ep_arrive[i]);
      c.ep_tile_expected = reinterpret_cast<const uint32_t*>(cm->ep_tile_expected);
      c.n_copy = cm->n_copy > 0 ? cm->n_copy : 16;
      if (grid + c.n_copy > sms) grid = sms - c.n_copy;
      grid += c.n_copy;
      if (!bm) return BN == 256 ? launch_cfg<256, false, false, 3>(kp, grid, st) : launch_cfg<128, false, false, 3>(kp, grid, st);
      return BN == 256 ? launch_cfg<256, false, true, 3>(kp, grid, st) : launch_cfg<128, false, true, 3>(kp, grid, st);
    }
    return -33;
  }
  if (BN == 256) {
    if (!am && !bm) return launch_cfg<256, false, false>(kp, grid, st);
    if (!am && bm) return launch_cfg<256, false, true>(kp, grid, st);
    if (am && !bm) return launch_cfg<256, true, false>(kp, grid, st);
    return launch_cfg<256, true, true>(kp, grid, st);
  } else {
    if (!am && !bm) return launch_cfg<128, false, false>(kp, grid, st);
    if (!am && bm) return launch_cfg<128, false, true>(kp, grid, st);
    if (am && !bm) return launch_cfg<128, true, false>(kp, grid, st);
    return launch_cfg<128, true, true>(kp, grid, st);
  }
}

extern "C" int sx_gemm_bf16(const SxGemmArgs* a, cudaStream_t st) { return gemm_launch(a, nullptr, st); }

// F2 / F3 / F4: the same GEMM with a collective fused in (see CommParams above and SxGemmCommArgs in sx_api.h).
extern "C" int sx_gemm_bf16_comm(const SxGemmArgs* a, const SxGemmCommArgs* cm, cudaStream_t st) {
  if (!cm) return -30;
  return gemm_launch(a, cm, st);
}
