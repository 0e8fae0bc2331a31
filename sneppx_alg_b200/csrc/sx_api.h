// C ABI of the sm_100a kernel library. Every entry point takes raw device pointers and a stream,
// returns 0 on success (negative: argument / launch error) and never allocates device memory
// unless its comment says so. Kernels that can wait (mbarrier pipelines, peer signals) take a
// `status` word in device memory: 0 = ok, otherwise one of the sx::ST_* codes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ------------------------------------------------------------------ G1 / G2 GEMM
typedef struct SxGemmArgs {
  const void* A;      // a_mn == 0: [M, K] row-major (lda);  a_mn == 1: [K, M] row-major (lda)
  const void* B;      // b_mn == 0: [N, K] row-major (ldb);  b_mn == 1: [K, N] row-major (ldb)
  void* D;            // [M, N] row-major (ldd), bf16 or fp32
  const void* C;      // optional addend, same indexing as D (ldc), bf16 or fp32
  const float* bias;  // optional [N]
  int M, N, K, batch;
  long long lda, ldb, ldd, ldc;
  long long strideA, strideB, strideD, strideC;  // batch strides in elements (0: operand shared)
  int a_mn, b_mn;
  int out_fp32, c_fp32;
  int act;  // 0 none, 1 gelu(tanh), 2 silu, 3 relu
  float alpha, beta;
  const int* tile_group;  // grouped GEMM: per 128-row block of A, index of the B matrix (-1 skips the block)
  int num_groups;         // number of B matrices when tile_group is set
  const int* k_ranges;    // per batch [k_begin, k_end) rows of the MN-major operands to reduce over
  int k_total;            // total rows of the MN-major operands when k_ranges is set
  int* status;
  int sm_limit;  // cap on CTAs (0: one per SM)
  int force_bn;  // 0 auto, 128 or 256
  int flags;     // bit 0: B is not written by any kernel launched before this one on the stream (a weight at
                 // inference time), so a kernel may start fetching it before its predecessor has finished
} SxGemmArgs;
int sx_gemm_bf16(const SxGemmArgs* args, cudaStream_t stream);

// ------------------------------------------------------------------ A1 / A2 flash attention
// Q [B, Sq, Hq, D], K [B, Skv, Hk, D], V [B, Skv, Hk / v_head_div, D], O [B, Sq, Hq, D]; bf16; each given as a
// base pointer plus token (row) and batch strides in elements, so slices of a fused QKV buffer work in place.
typedef struct SxAttnArgs {
  const void* Q; const void* K; const void* V; void* O;
  float* lse;              // [B, Hq, Sq] natural-log LSE (forward: out; backward: in)
  const void* dO;          // backward only
  void* dQ; void* dK; void* dV;  // backward outputs (bf16), same strides as Q / K / V
  float* dq_accum;         // backward scratch: [B, Sq, Hq, D] fp32, zero-filled by the call
  float* delta;            // backward scratch: [B, Hq, Sq] fp32
  long long q_row_stride, k_row_stride, v_row_stride, o_row_stride;
  long long q_batch_stride, k_batch_stride, v_batch_stride;
  long long do_row_stride, dq_row_stride, dk_row_stride, dv_row_stride;
  long long dq_batch_stride, dk_batch_stride, dv_batch_stride;
  int B, Sq, Skv, Hq, Hk, D;
  int v_head_div;          // 1; 2 for differential attention (two score heads share a V head)
  int causal, window;
  float scale;
  int* status;
  // forward only: optional byte per 128 x 128 score tile, [B or 1][Hq or 1][ceil(Sq/128)][ceil(Skv/128)]; a zero
  // byte removes the tile. Strides in bytes (0 = shared over the batch / the heads).
  const void* block_mask;
  long long bm_batch_stride, bm_head_stride;
} SxAttnArgs;
int sx_attn_fwd(const SxAttnArgs* args, cudaStream_t stream);
int sx_attn_bwd(const SxAttnArgs* args, cudaStream_t stream);

// ------------------------------------------------------------------ fused collectives over symmetric memory
// Peer tables hold, for every rank of the group, the peer-mapped address of the same symmetric allocation.
// `pad` is the group's signal pad (uint32 words, zero-initialised once). Every wait inside these kernels is
// bounded by timeout_ns and reports through `status`.
typedef struct SxPeers {
  void* buf[8];
  void* pad[8];
  int rank, world;
  unsigned long long timeout_ns;
} SxPeers;

// Barrier across the group on `channel` (epoch must increase by one per call on that channel).
int sx_peer_barrier(const SxPeers* peers, int channel, unsigned epoch, int* status, cudaStream_t stream);

// F1, ZeRO gradient reduce-scatter fused with the partitioned optimizer.
//   peers->buf[r]  : rank r's flat bf16 gradient buffer (all ranks hold the full bucket)
//   elem_offset/n  : this rank's shard of the bucket, in elements (n % 8 == 0, offset % 8 == 0)
//   mode 1 (reduce): reduced = (sum_r grad_r) / world -> `reduced` (fp32, local, indexed from 0), per-CTA
//                    sum-of-squares partials -> sumsq_partials[0..grid) ; waits for every rank's `ready_epoch`
//                    on channel `ready_channel` first (peers signal it when their bucket is complete).
//   mode 2 (update): exchanges this rank's total sum of squares with all peers (channel norm_channel), derives the
//                    clip coefficient from the global norm, runs AdamW on (p32, m, v) with `reduced` and writes
//                    the bf16 shard to p16_out; ends with a barrier on channel done_channel.
//   mode 3 (fused) : no clipping: reduce + AdamW in one pass, nothing stored in between; same start / end barriers.
typedef struct SxZeroArgs {
  SxPeers peers;
  long long elem_offset, n;
  float* reduced;            // fp32 [n] (modes 1, 2)
  float* sumsq_partials;     // fp32 [num_partials] (mode 1 writes `grid` entries at partial_offset; mode 2 reads all)
  int partial_offset, num_partials;
  float* p32; float* m; float* v; void* p16_out;
  float lr, beta1, beta2, eps, wd; int step;
  float max_norm;            // <= 0: no clipping
  float* norm_out;           // [3] {sum of squares, norm, coefficient}
  int ready_channel; unsigned ready_epoch;
  int norm_channel; unsigned norm_epoch;
  int done_channel; unsigned done_epoch;
  int mode;
  int grid;                  // CTAs to use (0: default)
  int* status;
  const void* mc_buf;        // optional: NVLS multicast mapping of the gradient buffer (same layout as peers.buf[r]).
                             // When set, modes 1 and 3 read each 16 bytes with ONE multimem.ld_reduce (the switch sums
                             // the ranks' values in fp32 and returns bf16) instead of `world` peer loads.
} SxZeroArgs;
int sx_zero_grid_default(void);
int sx_zero_step(const SxZeroArgs* args, cudaStream_t stream);
// Tell all peers that this rank's bucket is complete (one tiny launch on the stream that produced the gradients).
int sx_signal_peers(const SxPeers* peers, int channel, unsigned epoch, cudaStream_t stream);

// F2 (copy form): pull every rank's shard [n elements of `elem_bytes`] into dst[r * n ...] over NVLink.
// Waits for `epoch` on `channel` from every rank first when channel >= 0.
int sx_allgather_pull(const SxPeers* peers, void* dst, long long shard_bytes, long long src_offset_bytes, int channel,
                      unsigned epoch, int grid, int* status, cudaStream_t stream);

// One-shot all-reduce of bf16 activations (tensor-parallel decode / short prefill): out = sum over ranks of their
// staging buffers (peers->buf[r], n values each, n % 8 == 0). The epoch lives in device memory (epoch_ctr, advanced
// by the launch), so the launch can be captured in a CUDA graph. Channels `channel`, `channel + 1`.
int sx_allreduce_bf16(const SxPeers* peers, void* out, long long n, int channel, void* epoch_ctr, void* cta_counter,
                      int grid, int* status, cudaStream_t stream);

// F2 (push form, NVLS): every rank stores its shard ONCE to the multicast mapping of the full-size symmetric buffer
// (multimem.st: the switch delivers it to all ranks), then the grid's last CTA signals `channel` = `epoch` to every rank
// and waits for every rank's signal, so when the kernel ends on a rank, all shards have landed in its copy.
// mc_dst: multicast address of this rank's slot in the full buffer. Callers must make sure no rank still reads the old
// contents of the buffer when any rank starts pushing (the ZeRO engine's optimizer kernel ends with such a barrier).
int sx_allgather_mc(const SxPeers* peers, const void* src_shard, void* mc_dst, long long shard_bytes, int channel,
                    unsigned epoch, int grid, int* status, cudaStream_t stream);
// Link micro-benchmark kernels: move / reduce `bytes` through peer loads, peer stores, multimem.ld_reduce or multimem.st.
//   kind 0: pull   dst_local <- peers.buf[peer]          kind 1: push   peers.buf[peer] <- src_local
//   kind 2: NVLS ld_reduce over mc (bf16 sum) -> dst_local  kind 3: NVLS multimem.st  mc <- src_local
int sx_link_probe(const SxPeers* peers, int kind, int peer, const void* mc, void* local, long long bytes, int grid,
                  cudaStream_t stream);

// F2 / F3 / F4: GEMM with a collective fused into the same kernel.
//   mode 1  all-gather A rows -> GEMM   (TP column-parallel / sequence-parallel input; F3)
//   mode 2  all-gather B rows -> GEMM   (ZeRO-3 weight shards pulled by the consuming GEMM; F2)
//   mode 3  GEMM -> reduce-scatter of output rows (TP row-parallel output; F4)
// Modes 1/2: peers.buf[r] is rank r's copy of the full-size symmetric operand buffer, whose chunk r (chunk_rows rows)
// rank r has filled before the launch; the local copy is the GEMM operand (args->A or args->B must be
// peers.buf[rank]). flags: local uint32 [world * chunk_rows / sub_rows], zeroed once; epoch increases per call.
// Mode 3: peers.buf[r] is rank r's staging buffer, bf16 [world][chunk_rows][N]; rs_out [chunk_rows, N] (ld rs_ldd) gets
// the sum over ranks (+ rs_residual); counter_word: first of chunk_rows/128 words of the signal pad used as counters.
// The grid never exceeds the SM count: all CTAs of a launch are resident together, which the in-kernel waits rely on.
typedef struct SxGemmCommArgs {
  SxPeers peers;
  int mode;
  void* flags;
  unsigned epoch;
  int n_copy;
  int chunk_rows, sub_rows;
  int sig_channel, done_channel, counter_word;
  unsigned rs_expected;  // mode 3: counter value that marks a row block complete (previous value + 4 * ceil(N/BN) * world)
  void* rs_out; const void* rs_residual; long long rs_ldd;
  void* cta_counter;   // local uint32 word, zeroed once
  // mode 4 (F5): expert all-to-all dispatch fused with the grouped GEMM (args->tile_group must be set; args->A is
  // peers.buf[rank], the local expert-sorted row buffer that every rank pushes into). Entry e = (token e / ep_k,
  // choice e % ep_k) goes to row ep_dest_row[e] of rank ep_dest_rank[e] (-1: dropped), scaled by ep_row_scale[e]
  // when given. ep_arrive[r]: rank r's arrival counters (one uint32 per 128-row tile, symmetric memory);
  // ep_tile_expected: local cumulative arrival targets per tile.
  const void* ep_x; const int* ep_dest_rank; const int* ep_dest_row; const float* ep_row_scale;
  int ep_entries, ep_k, ep_d;
  void* ep_arrive[8];
  const void* ep_tile_expected;
} SxGemmCommArgs;
int sx_gemm_bf16_comm(const SxGemmArgs* args, const SxGemmCommArgs* comm, cudaStream_t stream);

// AR1: small all-reduce (sum) of fp32 values through the peers' buffers; n <= 4096. In place on peers->buf[rank].
int sx_allreduce_small(const SxPeers* peers, int n, int channel, unsigned epoch, int* status, cudaStream_t stream);

// ------------------------------------------------------------------ RNG, dropout, LayerNorm backward, FM / ARC steps
// Philox4x32-10 keyed by `seed`; element i of stream `offset` is the same whatever the launch geometry.
// mode 0 uniform [a, b), 1 normal(mean a, std b), 2 bernoulli(p = a) as 0 / 1. `out` 16-byte aligned.
int sx_rng_fill(float* out, long long n, int mode, float a, float b, unsigned long long seed, unsigned long long offset, cudaStream_t stream);
// bf16, n % 8 == 0: y = x * keep / (1 - p). Backward is the same call on dy with the same (seed, offset).
int sx_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, unsigned long long offset, cudaStream_t stream);
// LayerNorm backward: x, dy, dx bf16 [rows, cols]; gamma fp32; mean / rstd fp32 [rows] from sx_layernorm_fwd;
// partials fp32 [sx_layernorm_bwd_blocks(rows), 2, cols] scratch; dgamma_dbeta fp32 [2, cols]. cols % 8 == 0, <= 8192.
int sx_layernorm_bwd_blocks(long long rows);
int sx_layernorm_bwd(const void* x, const void* dy, const float* gamma, const float* mean, const float* rstd, void* dx,
                     float* partials, float* dgamma_dbeta, long long rows, int cols, cudaStream_t stream);
// Gradient compression (fp32): int8 with one scale per 256 values (n % 256 == 0); top-2 of every 32 values with the
// dropped part in `residual` (optional; n % 32 == 0); weighted sum of up to 16 equally sized buffers (n % 4 == 0).
int sx_fm_quant_int8(const float* x, void* q, float* scales, long long n, cudaStream_t stream);
int sx_fm_dequant_int8(const void* q, const float* scales, float* y, long long n, cudaStream_t stream);
int sx_fm_block_top2(const float* x, float* kept, float* residual, long long n, cudaStream_t stream);
int sx_fm_weighted_avg(const float* const* inputs, const float* weights, int count, float* out, long long n, cudaStream_t stream);
// Adversarial steps (fp32, n % 4 == 0). mode 0 FGSM, 1 PGD step with projection onto the eps-ball around x0,
// 2 sine obfuscation x + eps * sin(100 x), 3 Gaussian smoothing sample x + eps * N(0, 1).
int sx_arc_step(const float* x, const float* g, const float* x0, float* out, long long n, int mode, float eps, float alpha,
                float lo, float hi, unsigned long long seed, unsigned long long offset, cudaStream_t stream);

// conv2d backward: x [N,C,H,W], w [K,C,R,S], dy [N,K,OH,OW] (fp32, or bf16 with is_bf16), contiguous; fp32 gradients
// dx / dw / db, any of which may be null to skip it.
int sx_conv2d_bwd(const void* x, const void* w, const void* dy, float* dx, float* dw, float* db, int N, int C, int H, int W,
                  int K, int R, int S, int stride, int pad, int is_bf16, cudaStream_t stream);

// NPE bytecode interpreter: instruction table [n, 8] int32 (op, dest, a, b, immediate, rows, cols, bias register);
// program memory and x / out fp32. The planner returns 0, -1 malformed, -2 shapes do not fit, -3 unsupported opcode.
int sx_npe_plan_program(const int* prog8, int n, long long mem_size, int in_w, int* maxw, int* out_w);
int sx_npe_run(const int* prog_host, const int* prog_dev, int n, const float* mem, long long mem_size, const float* x, long long rows,
               int in_w, float* out, int out_w_expected, cudaStream_t stream);

// Block-scaled fp8 (e4m3) GEMM, y = (xq * sx) (wq * sw)^T: xq [M, K] with fp32 scales sx [M, K/128] (1 x 128 blocks),
// wq [N, K] with sw [ceil(N/128), K/128] (128 x 128 blocks), bf16 out. `work`: sx_gemm_fp8_workspace bytes (or null).
long long sx_gemm_fp8_workspace(int M, int N, int K);
int sx_gemm_fp8(const void* xq, long long ldx, const float* sx, const void* wq, long long ldw, const float* sw,
                const float* bias, void* out, long long ldd, float* work, int M, int N, int K, int* status,
                cudaStream_t stream);
// Grouped form for SER experts: expert-sorted token rows (segments padded to 128 rows) times the stacked expert
// weights [E * N, K] (N % 128 == 0, scales [E * N/128, K/128]); tile_group[t] is the expert of token tile t
// (-1: unused tile, its output rows are zero).
int sx_gemm_fp8_grouped(const void* xq, long long ldx, const float* sx, const void* wq, long long ldw, const float* sw,
                        const int* tile_group, int num_experts, void* out, long long ldd, int rows, int N, int K,
                        int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
