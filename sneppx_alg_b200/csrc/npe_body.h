// Row-wise interpreter for NPE bytecode, shared by the CUDA kernel (npe_interp.cu) and the CPU oracle
// (host/cpu_oracle.cpp): the planner that checks a program and sizes its registers, and the executor of one input row.
//
// A program sees its input x [rows, width] in register 0 and runs once per row; every register holds either a vector
// of that row (in the caller's scratch, `maxw` floats per slot) or a matrix that stays in program memory. Supported:
// LOAD / STORE / NOP / HALT, elementwise arithmetic, the unary functions, MATMUL and FUSED_LINEAR of a row with a
// matrix [in, out], SOFTMAX and LAYERNORM over the row, DROPOUT (identity), CONCAT and SPLIT. Programs that need other
// rows (ATTENTION), data-dependent control flow (BRANCH) or index inputs are refused by the planner with code -3 and
// stay on the host VM.
#pragma once

#include <math.h>

#if defined(__CUDACC__)
#define SX_NPE_HD __host__ __device__ __forceinline__
#else
#define SX_NPE_HD inline
#endif

enum {
  NPE_NOP = 0, NPE_LOAD = 1, NPE_STORE = 2, NPE_ADD = 3, NPE_SUB = 4, NPE_MUL = 5, NPE_DIV = 6, NPE_MATMUL = 7, NPE_RELU = 8,
  NPE_SOFTMAX = 9, NPE_LAYERNORM = 10, NPE_HALT = 13, NPE_NEG = 14, NPE_EXP = 15, NPE_LOG = 16, NPE_SQRT = 17, NPE_POW = 18,
  NPE_SIN = 19, NPE_COS = 20, NPE_TANH = 21, NPE_SIGMOID = 22, NPE_GELU = 23, NPE_SILU = 24, NPE_DROPOUT = 25, NPE_CONCAT = 32,
  NPE_SPLIT = 33, NPE_FUSED_LINEAR = 40
};
#define SX_NPE_REGS 16

struct SxNpeIns { int op, dest, a, b, imm, rows, cols, bias_reg; };   // rows / cols: shape_a; bias_reg: shape_b[0]

SX_NPE_HD bool sx_npe_is_unary(int op) {
  return op == NPE_RELU || op == NPE_NEG || op == NPE_EXP || op == NPE_LOG || op == NPE_SQRT || op == NPE_SIN || op == NPE_COS ||
         op == NPE_TANH || op == NPE_SIGMOID || op == NPE_GELU || op == NPE_SILU || op == NPE_DROPOUT;
}
SX_NPE_HD bool sx_npe_is_binary(int op) { return op == NPE_ADD || op == NPE_SUB || op == NPE_MUL || op == NPE_DIV || op == NPE_POW; }

SX_NPE_HD float sx_npe_unary(int op, float v) {
  switch (op) {
    case NPE_RELU: return v > 0.f ? v : 0.f;
    case NPE_NEG: return -v;
    case NPE_EXP: return expf(v);
    case NPE_LOG: return logf(v);
    case NPE_SQRT: return sqrtf(v);
    case NPE_SIN: return sinf(v);
    case NPE_COS: return cosf(v);
    case NPE_TANH: return tanhf(v);
    case NPE_SIGMOID: return 1.f / (1.f + expf(-v));
    case NPE_GELU: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case NPE_SILU: return v / (1.f + expf(-v));
    default: return v;   // DROPOUT at inference, and activation code 0
  }
}
SX_NPE_HD float sx_npe_binary(int op, float x, float y) {
  switch (op) {
    case NPE_ADD: return x + y;
    case NPE_SUB: return x - y;
    case NPE_MUL: return x * y;
    case NPE_DIV: return x / y;
    default: return powf(x, y);
  }
}

// Walks the program once with register widths only. Returns 0 and the widest vector / the output width, or
// -1 malformed instruction, -2 shapes that do not fit, -3 an instruction this interpreter does not run.
inline int sx_npe_plan(const SxNpeIns* prog, int n, long long mem_size, int in_w, int* maxw, int* out_w) {
  int kind[SX_NPE_REGS] = {0}, width[SX_NPE_REGS] = {0}, mrows[SX_NPE_REGS] = {0};   // kind 0 empty, 1 vector, 2 matrix
  kind[0] = 1; width[0] = in_w;
  int widest = in_w, result = -1, last = in_w;
  for (int pc = 0; pc < n; ++pc) {
    const SxNpeIns& i = prog[pc];
    if (i.dest < 0 || i.dest >= SX_NPE_REGS || i.a < 0 || i.a >= SX_NPE_REGS || i.b < 0 || i.b >= SX_NPE_REGS) return -1;
    int w = -1;
    if (i.op == NPE_HALT) break;
    if (i.op == NPE_NOP) continue;
    if (i.op == NPE_LOAD) {
      const long long count = i.cols ? (long long)i.rows * i.cols : i.rows;
      if (i.rows < 1 || i.cols < 0 || i.imm < 0 || i.imm + count > mem_size) return -2;
      if (i.cols) { kind[i.dest] = 2; mrows[i.dest] = i.rows; width[i.dest] = i.cols; continue; }
      w = i.rows;
    } else if (i.op == NPE_STORE) {
      if (kind[i.a] != 1) return -2;
      result = width[i.a];
      continue;
    } else if (i.op == NPE_MATMUL || i.op == NPE_FUSED_LINEAR) {
      if (kind[i.a] != 1) return -2;
      if (kind[i.b] == 2) {
        if (mrows[i.b] != width[i.a]) return -2;
        w = width[i.b];
      } else if (kind[i.b] == 1 && i.op == NPE_MATMUL) {
        if (width[i.b] != width[i.a]) return -2;
        w = width[i.a];
      } else return -2;
      if (i.op == NPE_FUSED_LINEAR) {
        if (i.bias_reg < 0 || i.bias_reg >= SX_NPE_REGS || kind[i.bias_reg] != 1 || width[i.bias_reg] != w) return -2;
        if (i.imm != 0 && !sx_npe_is_unary(i.imm)) return -3;
      }
    } else if (sx_npe_is_unary(i.op) || i.op == NPE_SOFTMAX || i.op == NPE_LAYERNORM) {
      if (kind[i.a] != 1) return -2;
      w = width[i.a];
    } else if (sx_npe_is_binary(i.op)) {
      if (kind[i.a] != 1 || kind[i.b] != 1 || width[i.a] != width[i.b]) return -2;
      w = width[i.a];
    } else if (i.op == NPE_CONCAT) {
      if (kind[i.a] != 1 || kind[i.b] != 1) return -2;
      w = width[i.a] + width[i.b];
    } else if (i.op == NPE_SPLIT) {
      if (kind[i.a] != 1 || width[i.a] % 2) return -2;
      w = width[i.a] / 2;
    } else {
      return -3;
    }
    kind[i.dest] = 1; width[i.dest] = w; last = w;
    if (w > widest) widest = w;
  }
  *maxw = widest;
  *out_w = result >= 0 ? result : last;
  return 0;
}

// Runs a planned program on one row. `slots`: (SX_NPE_REGS + 1) * maxw floats private to the row (the extra slot is
// scratch for results that may overwrite their own operand). Ctx: tid(), nthreads(), sync(), sum(v), max(v) over the
// threads that share the row (one thread on the host, one block on the device).
template <class Ctx>
SX_NPE_HD void sx_npe_exec_row(const SxNpeIns* prog, int n, const float* mem, const float* x_row, int in_w, float* out_row,
                               float* slots, int maxw, Ctx& ctx) {
  int width[SX_NPE_REGS], mrows[SX_NPE_REGS];
  const float* mat[SX_NPE_REGS];
  for (int r = 0; r < SX_NPE_REGS; ++r) { width[r] = 0; mrows[r] = 0; mat[r] = nullptr; }
  float* scratch = slots + (long long)SX_NPE_REGS * maxw;
  const int tid = ctx.tid(), nt = ctx.nthreads();
  for (int j = tid; j < in_w; j += nt) slots[j] = x_row[j];
  width[0] = in_w;
  ctx.sync();
  int result = -1, last = 0;
  for (int pc = 0; pc < n; ++pc) {
    const SxNpeIns i = prog[pc];
    if (i.op == NPE_HALT) break;
    if (i.op == NPE_NOP) continue;
    if (i.op == NPE_STORE) {                     // the value at this moment is the result, whatever the register holds later
      for (int j = tid; j < width[i.a]; j += nt) out_row[j] = slots[(long long)i.a * maxw + j];
      result = i.a;
      continue;
    }
    const float* va = slots + (long long)i.a * maxw;
    const float* vb = slots + (long long)i.b * maxw;
    float* vd = slots + (long long)i.dest * maxw;
    int w = 0;
    if (i.op == NPE_LOAD) {
      if (i.cols) { mat[i.dest] = mem + i.imm; mrows[i.dest] = i.rows; width[i.dest] = i.cols; continue; }
      w = i.rows;
      for (int j = tid; j < w; j += nt) scratch[j] = mem[i.imm + j];
    } else if (i.op == NPE_MATMUL || i.op == NPE_FUSED_LINEAR) {
      if (mat[i.b] != nullptr && mrows[i.b] == width[i.a]) {
        w = width[i.b];
        const float* M = mat[i.b];
        const float* bias = i.op == NPE_FUSED_LINEAR ? slots + (long long)i.bias_reg * maxw : nullptr;
        for (int j = tid; j < w; j += nt) {
          float acc = bias ? bias[j] : 0.f;
          for (int k = 0; k < width[i.a]; ++k) acc += va[k] * M[(long long)k * w + j];
          scratch[j] = i.op == NPE_FUSED_LINEAR ? sx_npe_unary(i.imm, acc) : acc;
        }
      } else {
        w = width[i.a];
        for (int j = tid; j < w; j += nt) scratch[j] = va[j] * vb[j];
      }
    } else if (i.op == NPE_SOFTMAX) {
      w = width[i.a];
      float m = -INFINITY;
      for (int j = tid; j < w; j += nt) m = fmaxf(m, va[j]);
      m = ctx.max(m);
      float s = 0.f;
      for (int j = tid; j < w; j += nt) { const float e = expf(va[j] - m); scratch[j] = e; s += e; }
      s = ctx.sum(s);
      for (int j = tid; j < w; j += nt) scratch[j] /= s;
    } else if (i.op == NPE_LAYERNORM) {
      w = width[i.a];
      float s = 0.f;
      for (int j = tid; j < w; j += nt) s += va[j];
      const float mean = ctx.sum(s) / (float)w;
      float q = 0.f;
      for (int j = tid; j < w; j += nt) { const float d = va[j] - mean; q += d * d; }
      const float rstd = 1.f / sqrtf(ctx.sum(q) / (float)w + 1e-5f);
      for (int j = tid; j < w; j += nt) scratch[j] = (va[j] - mean) * rstd;
    } else if (i.op == NPE_CONCAT) {
      w = width[i.a] + width[i.b];
      for (int j = tid; j < w; j += nt) scratch[j] = j < width[i.a] ? va[j] : vb[j - width[i.a]];
    } else if (i.op == NPE_SPLIT) {
      w = width[i.a] / 2;
      for (int j = tid; j < w; j += nt) scratch[j] = va[(i.imm & 1) * w + j];
    } else if (sx_npe_is_binary(i.op)) {
      w = width[i.a];
      for (int j = tid; j < w; j += nt) scratch[j] = sx_npe_binary(i.op, va[j], vb[j]);
    } else {
      w = width[i.a];
      for (int j = tid; j < w; j += nt) scratch[j] = sx_npe_unary(i.op, va[j]);
    }
    ctx.sync();                                   // every operand has been read before the destination changes
    for (int j = tid; j < w; j += nt) vd[j] = scratch[j];
    width[i.dest] = w; mat[i.dest] = nullptr; mrows[i.dest] = 0;
    last = i.dest;
    ctx.sync();
  }
  if (result < 0)
    for (int j = tid; j < width[last]; j += nt) out_row[j] = slots[(long long)last * maxw + j];
}
