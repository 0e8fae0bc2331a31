// Edge runtime: bump arena, fp32 / int8 kernels (matmul, 2-D convolution, relu) and a tiny op-code interpreter for
// "EDGE" model files (edge/src/edge_runtime.c of the reference defines the arena and relu and only declares matmul
// and conv; edge/sneppx-to-edge.py:9-19 gives the header + op-code file layout).
// File layout: "EDGE" u32 version u32 n_ops, then per op: u32 code (1 matmul, 2 relu, 3 add_bias), u32 rows, u32 cols,
// followed by rows*cols fp32 weights for matmul / cols fp32 for bias.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

namespace {
struct Arena {
  uint8_t* base;
  size_t cap, off;
};
struct Op {
  uint32_t code, rows, cols;
  std::vector<float> w;
};
struct EdgeModel {
  std::vector<Op> ops;
};
}  // namespace

extern "C" {
void* sx_edge_arena_create(size_t bytes) {
  Arena* a = new Arena{(uint8_t*)aligned_alloc(64, (bytes + 63) / 64 * 64), bytes, 0};
  return a;
}
void* sx_edge_arena_alloc(void* h, size_t bytes) {
  Arena* a = static_cast<Arena*>(h);
  size_t o = (a->off + 63) / 64 * 64;
  if (o + bytes > a->cap) return nullptr;
  a->off = o + bytes;
  return a->base + o;
}
void sx_edge_arena_reset(void* h) { static_cast<Arena*>(h)->off = 0; }
size_t sx_edge_arena_used(void* h) { return static_cast<Arena*>(h)->off; }
void sx_edge_arena_destroy(void* h) {
  Arena* a = static_cast<Arena*>(h);
  free(a->base);
  delete a;
}

void sx_edge_relu(float* x, size_t n) {
  for (size_t i = 0; i < n; ++i) x[i] = x[i] > 0 ? x[i] : 0;
}
// C[M,N] = A[M,K] * B[K,N]
void sx_edge_matmul(const float* A, const float* B, float* C, int M, int K, int N) {
  for (int i = 0; i < M; ++i) {
    float* c = C + (size_t)i * N;
    std::fill(c, c + N, 0.f);
    for (int k = 0; k < K; ++k) {
      const float a = A[(size_t)i * K + k];
      const float* b = B + (size_t)k * N;
      for (int j = 0; j < N; ++j) c[j] += a * b[j];
    }
  }
}
// int8 x int8 -> int32 accumulate, dequantised with per-tensor scales
void sx_edge_matmul_int8(const int8_t* A, const int8_t* B, float* C, int M, int K, int N, float sa, float sb) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      int32_t acc = 0;
      for (int k = 0; k < K; ++k) acc += (int32_t)A[(size_t)i * K + k] * (int32_t)B[(size_t)k * N + j];
      C[(size_t)i * N + j] = acc * sa * sb;
    }
}
float sx_edge_quantize_int8(const float* x, int8_t* q, size_t n) {
  float amax = 0;
  for (size_t i = 0; i < n; ++i) amax = std::max(amax, std::fabs(x[i]));
  const float s = amax > 0 ? amax / 127.f : 1.f;
  for (size_t i = 0; i < n; ++i) q[i] = (int8_t)std::lrintf(std::max(-127.f, std::min(127.f, x[i] / s)));
  return s;
}
// NCHW valid convolution, stride 1: in [C,H,W], w [O,C,KH,KW], out [O,H-KH+1,W-KW+1]
void sx_edge_conv2d(const float* in, const float* w, const float* bias, float* out, int C, int H, int W, int O, int KH,
                    int KW) {
  const int OH = H - KH + 1, OW = W - KW + 1;
  for (int o = 0; o < O; ++o)
    for (int y = 0; y < OH; ++y)
      for (int x = 0; x < OW; ++x) {
        float acc = bias ? bias[o] : 0.f;
        for (int c = 0; c < C; ++c)
          for (int ky = 0; ky < KH; ++ky)
            for (int kx = 0; kx < KW; ++kx)
              acc += in[((size_t)c * H + y + ky) * W + x + kx] * w[(((size_t)o * C + c) * KH + ky) * KW + kx];
        out[((size_t)o * OH + y) * OW + x] = acc;
      }
}

void* sx_edge_load(const char* path) {
  FILE* f = fopen(path, "rb");
  if (!f) return nullptr;
  char magic[4];
  uint32_t ver = 0, n = 0;
  if (fread(magic, 1, 4, f) != 4 || memcmp(magic, "EDGE", 4) || fread(&ver, 4, 1, f) != 1 || fread(&n, 4, 1, f) != 1 ||
      n > 4096) {
    fclose(f);
    return nullptr;
  }
  long here = ftell(f);
  fseek(f, 0, SEEK_END);
  const long file_end = ftell(f);
  fseek(f, here, SEEK_SET);
  EdgeModel* m = new EdgeModel();
  for (uint32_t i = 0; i < n; ++i) {
    Op op;
    if (fread(&op.code, 4, 1, f) != 1 || fread(&op.rows, 4, 1, f) != 1 || fread(&op.cols, 4, 1, f) != 1) break;
    if (op.code < 1 || op.code > 3) break;
    const size_t cnt = op.code == 1 ? (size_t)op.rows * op.cols : (op.code == 3 ? op.cols : 0);
    const long left = file_end - ftell(f);
    if (left < 0 || cnt > (size_t)left / 4) break;  // the weights must be in the file: no allocation from a bare header
    op.w.resize(cnt);
    if (cnt && fread(op.w.data(), 4, cnt, f) != cnt) break;
    m->ops.push_back(std::move(op));
  }
  fclose(f);
  if (m->ops.size() != n) { delete m; return nullptr; }
  return m;
}
// x: [batch, in_dim] -> returns output dim; y must hold batch * max layer width floats, as must scratch
int sx_edge_run(void* h, const float* x, int batch, int in_dim, float* y, float* scratch) {
  EdgeModel* m = static_cast<EdgeModel*>(h);
  std::vector<float> cur(x, x + (size_t)batch * in_dim), nxt;
  int dim = in_dim;
  (void)scratch;
  for (auto& op : m->ops) {
    if (op.code == 1) {
      if ((int)op.rows != dim) return -1;
      nxt.assign((size_t)batch * op.cols, 0.f);
      sx_edge_matmul(cur.data(), op.w.data(), nxt.data(), batch, dim, op.cols);
      cur.swap(nxt);
      dim = op.cols;
    } else if (op.code == 2) {
      sx_edge_relu(cur.data(), cur.size());
    } else if (op.code == 3) {
      if ((int)op.cols != dim) return -1;
      for (int b = 0; b < batch; ++b)
        for (int j = 0; j < dim; ++j) cur[(size_t)b * dim + j] += op.w[j];
    }
  }
  memcpy(y, cur.data(), cur.size() * sizeof(float));
  return dim;
}
// widest activation row the model produces for inputs of `in_dim` columns (the caller sizes `y` with it)
int sx_edge_max_width(void* h, int in_dim) {
  int w = in_dim;
  for (auto& op : static_cast<EdgeModel*>(h)->ops)
    if (op.code == 1 && (int)op.cols > w) w = (int)op.cols;
  return w;
}
void sx_edge_free(void* h) { delete static_cast<EdgeModel*>(h); }
}
