// Index arithmetic of the conv2d backward pass, shared by the CUDA kernels (conv2d_bwd.cu) and the CPU oracle
// (host/cpu_oracle.cpp), so that the arithmetic the GPU runs is the arithmetic the CPU tests check.
//
// Layouts: x [N, C, H, W], w [K, C, R, S], dy [N, K, OH, OW], all contiguous; OH = (H + 2 pad - R) / stride + 1.
#pragma once

#if defined(__CUDACC__)
#define SX_HD __host__ __device__ __forceinline__
#else
#define SX_HD inline
#endif

struct SxConvDims { int N, C, H, W, K, R, S, OH, OW, stride, pad; };

// dx[n, c, h, w] = sum over k, r, s of dy[n, k, (h + pad - r) / stride, (w + pad - s) / stride] * w[k, c, r, s]
// for the (r, s) whose offsets divide by the stride and land inside the output.
template <class Load>
SX_HD float sx_conv2d_dx_at(const SxConvDims& d, Load dy, Load wt, int n, int c, int h, int w) {
  float acc = 0.f;
  for (int r = 0; r < d.R; ++r) {
    const int th = h + d.pad - r;
    if (th < 0 || th % d.stride) continue;
    const int oh = th / d.stride;
    if (oh >= d.OH) continue;
    for (int s = 0; s < d.S; ++s) {
      const int tw = w + d.pad - s;
      if (tw < 0 || tw % d.stride) continue;
      const int ow = tw / d.stride;
      if (ow >= d.OW) continue;
      for (int k = 0; k < d.K; ++k)
        acc += dy((((long long)n * d.K + k) * d.OH + oh) * d.OW + ow) * wt((((long long)k * d.C + c) * d.R + r) * d.S + s);
    }
  }
  return acc;
}

// Partial sum of dw[k, c, r, s] over the flattened (n, oh, ow) positions first, first + step, ...
template <class Load>
SX_HD float sx_conv2d_dw_partial(const SxConvDims& d, Load dy, Load x, int k, int c, int r, int s, long long first, long long step) {
  float acc = 0.f;
  const long long total = (long long)d.N * d.OH * d.OW;
  for (long long i = first; i < total; i += step) {
    const int ow = (int)(i % d.OW), oh = (int)((i / d.OW) % d.OH), n = (int)(i / ((long long)d.OW * d.OH));
    const int h = oh * d.stride - d.pad + r, w = ow * d.stride - d.pad + s;
    if (h < 0 || h >= d.H || w < 0 || w >= d.W) continue;
    acc += dy((((long long)n * d.K + k) * d.OH + oh) * d.OW + ow) * x((((long long)n * d.C + c) * d.H + h) * d.W + w);
  }
  return acc;
}

// Partial sum of db[k] over the flattened (n, oh, ow) positions first, first + step, ...
template <class Load>
SX_HD float sx_conv2d_db_partial(const SxConvDims& d, Load dy, int k, long long first, long long step) {
  float acc = 0.f;
  const long long plane = (long long)d.OH * d.OW, total = (long long)d.N * plane;
  for (long long i = first; i < total; i += step) acc += dy(((i / plane) * d.K + k) * plane + i % plane);
  return acc;
}
