// S1/S2 support kernels of the chunked state-space-duality scan (Mamba-2 / HSS with diagonal A):
//   * build M = (C B^T) o L o dt per head from the group-shared C B^T (forward and backward),
//   * the backward pass over one Q x Q block: M, dG_h, row sums and column sums that give d(cumsum) and d(dt),
//   * the chunk-to-chunk state recurrence, forward and reversed,
//   * row-scaled copies and row dot products on the token-major [tokens, heads, headdim] layout.
// The GEMM-shaped parts run on the tcgen05 kernels (gemm_tc.cu, ssd_fwd.cu). The reference's scan is serial over
// the sequence (algorithms/hss/cuda/hss_cuda_extended.cu:27-77) and has no backward.
#include "common.cuh"
#include "sx_api.h"

namespace sx {

// ---------------------------------------------------------------------------------------------------------------
// One block per (batch*chunk, head). Vectors of 8 columns; Q/8 is a power of two <= 32, so a thread keeps the same
// column group for every row it visits (256 % (Q/8) == 0) and a row's vectors sit in adjacent lanes of one warp.
template <bool BWD>
__global__ void __launch_bounds__(256) ssd_qq_kernel(const __nv_bfloat16* __restrict__ dM, const float* __restrict__ CB,
                                                     const float* __restrict__ cs, const float* __restrict__ dt,
                                                     __nv_bfloat16* __restrict__ M, __nv_bfloat16* __restrict__ dGh,
                                                     float* __restrict__ rowW, float* __restrict__ colU, int H, int G,
                                                     int Q) {
  __shared__ float s_cs[256], s_dt[256], s_row[256], s_col[256];
  const long long bc = blockIdx.y;
  const int h = blockIdx.x, g = h / (H / G);
  const long long head = bc * H + h;
  const float* cb = CB + (bc * G + g) * (long long)Q * Q;
  for (int i = threadIdx.x; i < Q; i += 256) {
    s_cs[i] = cs[head * Q + i];
    s_dt[i] = dt[head * Q + i];
    s_col[i] = 0.f;
  }
  __syncthreads();
  const int vpr = Q >> 3;
  const int cg = threadIdx.x % vpr;
  const int s0 = cg * 8;
  float col[8], cs_s[8], dt_s[8];   // the thread's eight columns stay the same for every row it visits
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    col[j] = 0.f;
    cs_s[j] = s_cs[s0 + j];
    dt_s[j] = s_dt[s0 + j];
  }
  const long long base = head * (long long)Q * Q;
  for (int l = threadIdx.x / vpr; l < Q; l += 256 / vpr) {
    const long long off = base + (long long)l * Q + s0;
    float m[8], dg[8], rw = 0.f;
    if (s0 > l) {
#pragma unroll
      for (int j = 0; j < 8; ++j) m[j] = dg[j] = 0.f;
    } else {
      const float4 c0 = *reinterpret_cast<const float4*>(cb + (long long)l * Q + s0);
      const float4 c1 = *reinterpret_cast<const float4*>(cb + (long long)l * Q + s0 + 4);
      const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      float d[8];
      if (BWD) unpack8(ld8(dM + off), d);
      const float csl = s_cs[l];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int s = s0 + j;
        const float le = s <= l ? __expf(csl - cs_s[j]) : 0.f;
        const float lm = le * dt_s[j];
        m[j] = c[j] * lm;
        if (BWD) {
          dg[j] = d[j] * lm;
          const float u = d[j] * c[j] * le;
          col[j] += u;
          rw += u * dt_s[j];
        }
      }
    }
    st8(M + off, pack8(m));
    if (BWD) {
      st8(dGh + off, pack8(dg));
      for (int o = vpr >> 1; o > 0; o >>= 1) rw += __shfl_xor_sync(0xffffffffu, rw, o);
      if (cg == 0) s_row[l] = rw;
    }
  }
  if (BWD) {
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(&s_col[s0 + j], col[j]);
    __syncthreads();
    for (int i = threadIdx.x; i < Q; i += 256) {
      rowW[head * Q + i] = s_row[i];
      colU[head * Q + i] = s_col[i];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// State recurrence over chunks. One thread owns 8 consecutive elements of the [P*N] state of one (batch, head).
__global__ void __launch_bounds__(256) ssd_state_fwd_kernel(const float* __restrict__ S, const float* __restrict__ tot,
                                                            const float* __restrict__ init,
                                                            __nv_bfloat16* __restrict__ Hprev, float* __restrict__ fin,
                                                            int nc, int H, int PN) {
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int e = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (e >= PN) return;
  float st[8];
  if (init) {
    const float4 a = *reinterpret_cast<const float4*>(init + (long long)bh * PN + e);
    const float4 c = *reinterpret_cast<const float4*>(init + (long long)bh * PN + e + 4);
    st[0] = a.x; st[1] = a.y; st[2] = a.z; st[3] = a.w; st[4] = c.x; st[5] = c.y; st[6] = c.z; st[7] = c.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) st[j] = 0.f;
  }
#pragma unroll 4
  for (int c = 0; c < nc; ++c) {
    const long long o = (((long long)b * nc + c) * H + h) * PN + e;
    const float4 s0 = *reinterpret_cast<const float4*>(S + o);
    const float4 s1 = *reinterpret_cast<const float4*>(S + o + 4);
    const float t = tot[((long long)b * nc + c) * H + h];
    st8(Hprev + o, pack8(st));
    st[0] = st[0] * t + s0.x; st[1] = st[1] * t + s0.y; st[2] = st[2] * t + s0.z; st[3] = st[3] * t + s0.w;
    st[4] = st[4] * t + s1.x; st[5] = st[5] * t + s1.y; st[6] = st[6] * t + s1.z; st[7] = st[7] * t + s1.w;
  }
  float4* f = reinterpret_cast<float4*>(fin + (long long)bh * PN + e);
  f[0] = make_float4(st[0], st[1], st[2], st[3]);
  f[1] = make_float4(st[4], st[5], st[6], st[7]);
}

// Reverse: run = dfinal; for c = nc-1..0: dS_c = run; dtot_c = <run, H_c>; run = tot_c run + dHprev_c.
// PN is covered by gridDim.x blocks of 2048 elements; each warp adds its part of dtot with one atomic per chunk (no
// block barrier inside the sequential loop).
__global__ void __launch_bounds__(256) ssd_state_bwd_kernel(const float* __restrict__ dHprev,
                                                            const float* __restrict__ tot,
                                                            const __nv_bfloat16* __restrict__ Hprev,
                                                            const float* __restrict__ dfin,
                                                            __nv_bfloat16* __restrict__ dS, float* __restrict__ dtot,
                                                            float* __restrict__ dinit, int nc, int H, int PN) {
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int e = (blockIdx.x * 256 + threadIdx.x) * 8;
  const bool live = e < PN;
  float run[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) run[j] = 0.f;
  if (live && dfin) {
    const float4 a = *reinterpret_cast<const float4*>(dfin + (long long)bh * PN + e);
    const float4 c = *reinterpret_cast<const float4*>(dfin + (long long)bh * PN + e + 4);
    run[0] = a.x; run[1] = a.y; run[2] = a.z; run[3] = a.w; run[4] = c.x; run[5] = c.y; run[6] = c.z; run[7] = c.w;
  }
#pragma unroll 2
  for (int c = nc - 1; c >= 0; --c) {
    const long long o = (((long long)b * nc + c) * H + h) * PN + e;
    float dot = 0.f;
    if (live) {
      float hp[8];
      unpack8(ld8(Hprev + o), hp);
      const float4 g0 = *reinterpret_cast<const float4*>(dHprev + o);
      const float4 g1 = *reinterpret_cast<const float4*>(dHprev + o + 4);
      const float t = tot[((long long)b * nc + c) * H + h];
      st8(dS + o, pack8(run));
#pragma unroll
      for (int j = 0; j < 8; ++j) dot += run[j] * hp[j];
      run[0] = run[0] * t + g0.x; run[1] = run[1] * t + g0.y; run[2] = run[2] * t + g0.z; run[3] = run[3] * t + g0.w;
      run[4] = run[4] * t + g1.x; run[5] = run[5] * t + g1.y; run[6] = run[6] * t + g1.z; run[7] = run[7] * t + g1.w;
    }
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) atomicAdd(dtot + ((long long)b * nc + c) * H + h, dot);
  }
  if (live) {
    float4* f = reinterpret_cast<float4*>(dinit + (long long)bh * PN + e);
    f[0] = make_float4(run[0], run[1], run[2], run[3]);
    f[1] = make_float4(run[4], run[5], run[6], run[7]);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Layouts of the [tokens, heads, P] tensors. Token-major row r = (bc * Q + q) * H + h. The operands of the GEMMs that
// fold the heads of a B / C group into one matrix dimension are kept group-first, [bc][G][Q][H/G][P], so that
// (bc, group) is one linear batch index; gf_row maps a token-major row to its group-first row (the identity for G = 1).
__device__ __forceinline__ long long gf_row(long long r, int H, int Q, int G) {
  const int rep = H / G;
  const int h = (int)(r % H);
  const long long t = r / H;
  return (((t / Q) * G + h / rep) * Q + (t % Q)) * rep + h % rep;
}

// out (group-first) = a (token-major, token stride ald) * scale[row]
__global__ void __launch_bounds__(256) ssd_scale_rows_kernel(const __nv_bfloat16* __restrict__ a,
                                                             const float* __restrict__ scale,
                                                             __nv_bfloat16* __restrict__ out, long long rows, int P,
                                                             int H, long long ald, int Q, int G) {
  const int vp = P >> 3;
  const long long total = rows * vp;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long r = i / vp;
    float f[8];
    unpack8(ld8(a + (r / H) * ald + (i % ((long long)H * vp)) * 8), f);
    const float s = scale[r];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= s;
    st8(out + (gf_row(r, H, Q, G) * vp + i % vp) * 8, pack8(f));
  }
}


// Row kernels on the token-major layout: row r = ((bc * Q) + q) * H + h holds P = 8 * vp elements (vp a power of
// two <= 32); the vp lanes of a row are adjacent, so row sums are shuffles inside a warp. `hf` is the index of the
// same row in the heads-first layout [bc][H][Q] that the per-head GEMMs write.
__device__ __forceinline__ float seg_sum(float v, int vp) {
  for (int o = vp >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// y = Yi (heads-first) + E[r] * Yoff + D[h] * x
__global__ void __launch_bounds__(256) ssd_combine_kernel(const __nv_bfloat16* __restrict__ Yi,
                                                          const __nv_bfloat16* __restrict__ Yoff,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ E, const float* __restrict__ D,
                                                          __nv_bfloat16* __restrict__ y, long long rows, int H, int Q,
                                                          int vp, long long xld, int G) {
  const long long total = rows * vp;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long r = i / vp;
    const int pv = (int)(i % vp);
    const int h = (int)(r % H);
    const long long t = r / H;
    const long long hf = ((t / Q) * H + h) * Q + (t % Q);
    float a[8], b[8], xv[8], o[8];
    unpack8(ld8(Yi + (hf * vp + pv) * 8), a);
    unpack8(ld8(Yoff + (gf_row(r, H, Q, G) * vp + pv) * 8), b);
    unpack8(ld8(x + t * xld + (h * vp + pv) * 8), xv);
    const float e = E[r], d = D ? D[h] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] + e * b[j] + d * xv[j];
    st8(y + i * 8, pack8(o));
  }
}

// dye = dy * E[r]; dcs_off[r] = sum_p dy E Yoff; ddrow[r] = sum_p dy x
__global__ void __launch_bounds__(256) ssd_bwd_rows1_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ Yoff,
                                                            const float* __restrict__ E,
                                                            __nv_bfloat16* __restrict__ dye, float* __restrict__ dcs,
                                                            float* __restrict__ ddrow, long long rows, int vp,
                                                            int H, long long xld, int Q, int G) {
  const long long total = rows * vp;
  const long long span = ((total + 255) / 256) * 256;   // whole warps stay in the loop together for the shuffles
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < span; i += gridDim.x * 256ll) {
    const bool live = i < total;
    const long long r = live ? i / vp : 0;
    float g[8], xv[8], yo[8], o[8], s1 = 0.f, s2 = 0.f;
    if (live) {
      unpack8(ld8(dy + i * 8), g);
      unpack8(ld8(x + (r / H) * xld + (i % ((long long)H * vp)) * 8), xv);
      const long long gi = (gf_row(r, H, Q, G) * vp + i % vp) * 8;
      unpack8(ld8(Yoff + gi), yo);
      const float e = E[r];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = g[j] * e;
        s1 += o[j] * yo[j];
        s2 += g[j] * xv[j];
      }
      st8(dye + gi, pack8(o));
    }
    s1 = seg_sum(s1, vp);
    s2 = seg_sum(s2, vp);
    if (live && (i % vp) == 0) {
      dcs[r] = s1;
      ddrow[r] = s2;
    }
  }
}

// dx = D[h] dy + decay[r] dxw + dxi (heads-first); ddecay[r] = sum_p dxw x
__global__ void __launch_bounds__(256) ssd_bwd_rows2_kernel(const __nv_bfloat16* __restrict__ dy,
                                                            const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ dxw,
                                                            const __nv_bfloat16* __restrict__ dxi,
                                                            const float* __restrict__ decay, const float* __restrict__ D,
                                                            __nv_bfloat16* __restrict__ dx, float* __restrict__ ddecay,
                                                            long long rows, int H, int Q, int vp, long long xld,
                                                            int G) {
  const long long total = rows * vp;
  const long long span = ((total + 255) / 256) * 256;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < span; i += gridDim.x * 256ll) {
    const bool live = i < total;
    const long long r = live ? i / vp : 0;
    float s = 0.f;
    if (live) {
      const int pv = (int)(i % vp);
      const int h = (int)(r % H);
      const long long t = r / H;
      const long long hf = ((t / Q) * H + h) * Q + (t % Q);
      float g[8], xv[8], a[8], b[8], o[8];
      unpack8(ld8(dy + i * 8), g);
      unpack8(ld8(x + t * xld + (h * vp + pv) * 8), xv);
      unpack8(ld8(dxw + (gf_row(r, H, Q, G) * vp + pv) * 8), a);
      unpack8(ld8(dxi + (hf * vp + pv) * 8), b);
      const float dc = decay[r], d = D ? D[h] : 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = d * g[j] + dc * a[j] + b[j];
        s += a[j] * xv[j];
      }
      st8(dx + i * 8, pack8(o));
    }
    s = seg_sum(s, vp);
    if (live && (i % vp) == 0) ddecay[r] = s;
  }
}

// Token-major [bc][Q][H][P] (token stride ild) -> heads-first [bc][H][Q][P]; 16 bytes per thread, both sides move
// whole P-element rows (128 bytes for headdim 64).
__global__ void __launch_bounds__(256) ssd_heads_first_kernel(const __nv_bfloat16* __restrict__ in, long long ild,
                                                              __nv_bfloat16* __restrict__ out, long long rows, int H,
                                                              int Q, int vp) {
  const long long total = rows * vp;
  for (long long o = blockIdx.x * 256ll + threadIdx.x; o < total; o += gridDim.x * 256ll) {
    const int pv = (int)(o % vp);
    const long long hf = o / vp;          // (bc * H + h) * Q + q
    const int q = (int)(hf % Q);
    const long long bh = hf / Q;
    const int h = (int)(bh % H);
    const long long t = (bh / H) * Q + q;
    st8(out + o * 8, ld8(in + t * ild + (h * vp + pv) * 8));
  }
}

// Gate of the Mamba-2 block: out = y * silu(z), z read in place from a wider row-major tensor (row stride zld).
__global__ void __launch_bounds__(256) gate_mul_fwd_kernel(const __nv_bfloat16* __restrict__ y,
                                                           const __nv_bfloat16* __restrict__ z, long long zld,
                                                           __nv_bfloat16* __restrict__ out, long long rows, int cv) {
  const long long total = rows * cv;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long r = i / cv;
    const int c = (int)(i % cv) * 8;
    float a[8], b[8];
    unpack8(ld8(y + i * 8), a);
    unpack8(ld8(z + r * zld + c), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] *= b[j] / (1.f + __expf(-b[j]));
    st8(out + i * 8, pack8(a));
  }
}
__global__ void __launch_bounds__(256) gate_mul_bwd_kernel(const __nv_bfloat16* __restrict__ g,
                                                           const __nv_bfloat16* __restrict__ y,
                                                           const __nv_bfloat16* __restrict__ z, long long zld,
                                                           __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dz,
                                                           long long rows, int cv) {
  const long long total = rows * cv;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += gridDim.x * 256ll) {
    const long long r = i / cv;
    const int c = (int)(i % cv) * 8;
    float gv[8], a[8], b[8], oy[8], oz[8];
    unpack8(ld8(g + i * 8), gv);
    unpack8(ld8(y + i * 8), a);
    unpack8(ld8(z + r * zld + c), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-b[j]));
      oy[j] = gv[j] * b[j] * sg;
      oz[j] = gv[j] * a[j] * sg * (1.f + b[j] * (1.f - sg));
    }
    st8(dy + i * 8, pack8(oy));
    st8(dz + i * 8, pack8(oz));
  }
}

}  // namespace sx

using namespace sx;

static bool qq_ok(int Q) { return Q >= 8 && Q <= 256 && (Q & (Q - 1)) == 0; }

extern "C" int sx_ssd_build_m(const void* CB, const void* cs, const void* dt, void* M, long long BC, int H, int G, int Q,
                              cudaStream_t st) {
  if (!qq_ok(Q) || H % G) return -1;
  if (BC == 0) return 0;
  ssd_qq_kernel<false><<<dim3(H, (unsigned)BC), 256, 0, st>>>(nullptr, (const float*)CB, (const float*)cs,
                                                              (const float*)dt, (__nv_bfloat16*)M, nullptr, nullptr,
                                                              nullptr, H, G, Q);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_bwd_qq(const void* dM, const void* CB, const void* cs, const void* dt, void* M, void* dGh,
                             void* rowW, void* colU, long long BC, int H, int G, int Q, cudaStream_t st) {
  if (!qq_ok(Q) || H % G) return -1;
  if (BC == 0) return 0;
  ssd_qq_kernel<true><<<dim3(H, (unsigned)BC), 256, 0, st>>>((const __nv_bfloat16*)dM, (const float*)CB,
                                                             (const float*)cs, (const float*)dt, (__nv_bfloat16*)M,
                                                             (__nv_bfloat16*)dGh, (float*)rowW, (float*)colU, H, G, Q);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_state_fwd(const void* S, const void* tot, const void* init, void* Hprev, void* fin, int B, int nc,
                                int H, int PN, cudaStream_t st) {
  if (PN % 8) return -1;
  ssd_state_fwd_kernel<<<dim3((PN / 8 + 255) / 256, B * H), 256, 0, st>>>(
      (const float*)S, (const float*)tot, (const float*)init, (__nv_bfloat16*)Hprev, (float*)fin, nc, H, PN);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_state_bwd(const void* dHprev, const void* tot, const void* Hprev, const void* dfin, void* dS,
                                void* dtot, void* dinit, int B, int nc, int H, int PN, cudaStream_t st) {
  if (PN % 8) return -1;
  ssd_state_bwd_kernel<<<dim3((PN / 8 + 255) / 256, B * H), 256, 0, st>>>(
      (const float*)dHprev, (const float*)tot, (const __nv_bfloat16*)Hprev, (const float*)dfin, (__nv_bfloat16*)dS,
      (float*)dtot, (float*)dinit, nc, H, PN);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

// `ald` (and `xld` below): elements between consecutive tokens of the bf16 input, >= H * P, a multiple of 8.
extern "C" int sx_ssd_scale_rows(const void* a, const void* scale, void* out, long long rows, int P, int H,
                                 long long ald, int Q, int G, cudaStream_t st) {
  if (P % 8 || ald % 8 || H % G) return -1;
  const long long total = rows * (P / 8);
  if (total == 0) return 0;
  const long long nb = (total + 255) / 256;
  ssd_scale_rows_kernel<<<(unsigned)(nb < 148 * 16 ? nb : 148 * 16), 256, 0, st>>>(
      (const __nv_bfloat16*)a, (const float*)scale, (__nv_bfloat16*)out, rows, P, H, ald, Q, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

static bool vp_ok(int P) { const int vp = P / 8; return P % 8 == 0 && vp >= 1 && vp <= 32 && (vp & (vp - 1)) == 0; }
static unsigned row_grid(long long total) {
  const long long nb = (total + 255) / 256;
  return (unsigned)(nb < 148 * 16 ? nb : 148 * 16);
}

extern "C" int sx_ssd_combine(const void* Yi, const void* Yoff, const void* x, const void* E, const void* D, void* y,
                              long long rows, int H, int Q, int P, long long xld, int G, cudaStream_t st) {
  if (!vp_ok(P) || xld % 8 || H % G) return -1;
  if (rows == 0) return 0;
  ssd_combine_kernel<<<row_grid(rows * (P / 8)), 256, 0, st>>>((const __nv_bfloat16*)Yi, (const __nv_bfloat16*)Yoff,
                                                                (const __nv_bfloat16*)x, (const float*)E,
                                                                (const float*)D, (__nv_bfloat16*)y, rows, H, Q, P / 8, xld, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_bwd_rows1(const void* dy, const void* x, const void* Yoff, const void* E, void* dye, void* dcs,
                                void* ddrow, long long rows, int P, int H, long long xld, int Q, int G,
                                cudaStream_t st) {
  if (!vp_ok(P) || xld % 8 || H % G) return -1;
  if (rows == 0) return 0;
  ssd_bwd_rows1_kernel<<<row_grid(rows * (P / 8)), 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                  (const __nv_bfloat16*)Yoff, (const float*)E,
                                                                  (__nv_bfloat16*)dye, (float*)dcs, (float*)ddrow, rows,
                                                                  P / 8, H, xld, Q, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_bwd_rows2(const void* dy, const void* x, const void* dxw, const void* dxi, const void* decay,
                                const void* D, void* dx, void* ddecay, long long rows, int H, int Q, int P,
                                long long xld, int G, cudaStream_t st) {
  if (!vp_ok(P) || xld % 8 || H % G) return -1;
  if (rows == 0) return 0;
  ssd_bwd_rows2_kernel<<<row_grid(rows * (P / 8)), 256, 0, st>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)dxw, (const __nv_bfloat16*)dxi,
      (const float*)decay,
      (const float*)D, (__nv_bfloat16*)dx, (float*)ddecay, rows, H, Q, P / 8, xld, G);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_gate_mul_fwd(const void* y, const void* z, long long zld, void* out, long long rows, int C,
                               cudaStream_t st) {
  if (C % 8 || zld % 8) return -1;
  if (rows == 0) return 0;
  gate_mul_fwd_kernel<<<row_grid(rows * (C / 8)), 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)z, zld,
                                                                 (__nv_bfloat16*)out, rows, C / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_gate_mul_bwd(const void* g, const void* y, const void* z, long long zld, void* dy, void* dz,
                               long long rows, int C, cudaStream_t st) {
  if (C % 8 || zld % 8) return -1;
  if (rows == 0) return 0;
  gate_mul_bwd_kernel<<<row_grid(rows * (C / 8)), 256, 0, st>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)y,
                                                                 (const __nv_bfloat16*)z, zld, (__nv_bfloat16*)dy,
                                                                 (__nv_bfloat16*)dz, rows, C / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}

extern "C" int sx_ssd_heads_first(const void* in, long long ild, void* out, long long rows, int H, int Q, int P,
                                  cudaStream_t st) {
  if (P % 8 || ild % 8) return -1;
  if (rows == 0) return 0;
  ssd_heads_first_kernel<<<row_grid(rows * (P / 8)), 256, 0, st>>>((const __nv_bfloat16*)in, ild, (__nv_bfloat16*)out,
                                                                    rows, H, Q, P / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
