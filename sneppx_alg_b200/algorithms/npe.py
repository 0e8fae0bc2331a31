"""NPE — neural program engine: bytecode, register VM, verifier, compiler and JIT-style optimisation passes
(algorithms/npe/core/{program,vm,compiler,verify,jit_pipeline}.c; header neural_programming_engine.h:29-108;
CUDA interpreter npe_cuda.cu:23-117).

A program is a list of instructions over 16 tensor registers and one flat parameter memory.  The VM executes each
instruction as a batched device op (a MATMUL instruction is one tensor-core GEMM over the whole batch), so that a
compiled MLP costs two GEMM launches regardless of batch size; register 0 holds the input."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as tnn

from ..nn.modules import Module
from ..ops import functional as ops


class Op(enum.IntEnum):
    NOP = 0; LOAD = 1; STORE = 2; ADD = 3; SUB = 4; MUL = 5; DIV = 6; MATMUL = 7; RELU = 8; SOFTMAX = 9  # noqa: E702
    LAYERNORM = 10; ATTENTION = 11; BRANCH = 12; HALT = 13; NEG = 14; EXP = 15; LOG = 16; SQRT = 17; POW = 18  # noqa: E702
    SIN = 19; COS = 20; TANH = 21; SIGMOID = 22; GELU = 23; SILU = 24; DROPOUT = 25; CONV2D = 26; POOL2D = 27  # noqa: E702
    BATCHNORM = 28; EMBEDDING = 29; CROSSENTROPY = 30; MSE = 31; CONCAT = 32; SPLIT = 33  # noqa: E702
    FUSED_LINEAR = 40      # produced by the fusion pass: MATMUL + ADD (+ activation in ``immediate``)


NUM_REGS = 16
_UNARY = {Op.RELU: torch.relu, Op.NEG: torch.neg, Op.EXP: torch.exp, Op.LOG: torch.log, Op.SQRT: torch.sqrt,
          Op.SIN: torch.sin, Op.COS: torch.cos, Op.TANH: torch.tanh, Op.SIGMOID: torch.sigmoid,
          Op.GELU: tnn.functional.gelu, Op.SILU: tnn.functional.silu}
_BINARY = {Op.ADD: torch.add, Op.SUB: torch.sub, Op.MUL: torch.mul, Op.DIV: torch.div, Op.POW: torch.pow}


@dataclass
class Instruction:
    opcode: int
    dest: int = 0
    a: int = 0
    b: int = 0
    immediate: int = 0
    shape_a: tuple = (0, 0)
    shape_b: tuple = (0, 0)


@dataclass
class NPEConfig:
    """``SNEPPX_npe_config_default`` (program.c:28-43)."""
    max_program_length: int = 1024
    register_count: int = NUM_REGS
    step_limit: int = 10000
    verification_mode: int = 1
    trace_execution: bool = False
    jit_enabled: bool = True
    jit_hot_threshold: int = 100


class Program(Module):
    def __init__(self, memory_size=0, max_instructions=1024, device=None):
        super().__init__()
        self.instructions: List[Instruction] = []
        self.max_instructions = max_instructions
        self.memory = tnn.Parameter(torch.zeros(memory_size, device=device))

    def append(self, inst: Instruction):
        if len(self.instructions) >= self.max_instructions:
            raise OverflowError("program is full")
        self.instructions.append(inst)
        return self

    def clone_with(self, instructions):
        p = Program(0, self.max_instructions)
        p.memory = self.memory
        p.instructions = list(instructions)
        return p


def compile_mlp(dim, hidden, device=None, seed=0) -> Program:
    """x W1 + b1 -> ReLU -> W2 + b2 with the reference's memory layout (compiler.c:74-132):
    W1 [dim, hidden] at 0, b1 after it, then W2 [hidden, dim], b2, and an output slot."""
    o_b1 = dim * hidden
    o_w2 = o_b1 + hidden
    o_b2 = o_w2 + hidden * dim
    o_out = o_b2 + dim
    p = Program(o_out + dim, 32, device=device)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        p.memory[:o_b1] = (torch.randn(dim * hidden, generator=g) / dim ** 0.5).to(p.memory.device)
        p.memory[o_w2:o_b2] = (torch.randn(hidden * dim, generator=g) / hidden ** 0.5).to(p.memory.device)
    I = Instruction  # noqa: E741
    for inst in (I(Op.LOAD, 1, immediate=0, shape_a=(dim, hidden)), I(Op.LOAD, 2, immediate=o_b1, shape_a=(hidden, 0)),
                 I(Op.MATMUL, 3, 0, 1), I(Op.ADD, 4, 3, 2), I(Op.RELU, 5, 4),
                 I(Op.LOAD, 6, immediate=o_w2, shape_a=(hidden, dim)), I(Op.LOAD, 7, immediate=o_b2, shape_a=(dim, 0)),
                 I(Op.MATMUL, 8, 5, 6), I(Op.ADD, 9, 8, 7), I(Op.STORE, a=9, immediate=o_out), I(Op.HALT)):
        p.append(inst)
    return p


def compile_attention(seq_len, dim, device=None, seed=0) -> Program:
    """Single-head self-attention program (compiler.c:30-72): Q, K, V projections then the ATTENTION instruction."""
    p = Program(3 * dim * dim + seq_len * dim, 32, device=device)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        p.memory[: 3 * dim * dim] = (torch.randn(3 * dim * dim, generator=g) / dim ** 0.5).to(p.memory.device)
    I = Instruction  # noqa: E741
    for inst in (I(Op.LOAD, 1, immediate=0, shape_a=(dim, dim)), I(Op.LOAD, 2, immediate=dim * dim, shape_a=(dim, dim)),
                 I(Op.LOAD, 3, immediate=2 * dim * dim, shape_a=(dim, dim)), I(Op.MATMUL, 4, 0, 1), I(Op.MATMUL, 5, 0, 2),
                 I(Op.MATMUL, 6, 0, 3), I(Op.ATTENTION, 7, 4, 5, immediate=6), I(Op.STORE, a=7, immediate=3 * dim * dim),
                 I(Op.HALT)):
        p.append(inst)
    return p


def verify_program(prog: Program):
    """Static checks of verify.c:37-89. Returns (ok, messages)."""
    msgs, ok = [], True
    n = len(prog.instructions)
    if n == 0:
        return False, ["Program has no instructions"]
    for i, ins in enumerate(prog.instructions):
        if not (-1 <= ins.dest < NUM_REGS):
            msgs.append(f"Instr {i}: dest_reg {ins.dest} out of range [-1,15]")
            ok = False
        if ins.opcode in (Op.LOAD, Op.STORE) and not (0 <= ins.immediate < max(1, prog.memory.numel())):
            msgs.append(f"Instr {i}: address {ins.immediate} out of bounds [0,{prog.memory.numel()}]")
            ok = False
        if ins.opcode == Op.BRANCH:
            if not (0 <= ins.immediate < n):
                msgs.append(f"Instr {i}: branch target {ins.immediate} out of range [0,{n - 1}]")
                ok = False
            elif ins.immediate <= i:
                msgs.append(f"Instr {i}: backward branch may cause infinite loop")
    if prog.instructions[-1].opcode != Op.HALT:
        msgs.append("Warning: program does not end with HALT")
    return ok, msgs


@dataclass
class JITProfile:
    hot_threshold: int = 100
    op_frequency: dict = field(default_factory=dict)
    op_latency_us: dict = field(default_factory=dict)
    total_instructions: int = 0

    def record(self, opcode, latency_us):
        self.op_frequency[opcode] = self.op_frequency.get(opcode, 0) + 1
        self.op_latency_us[opcode] = self.op_latency_us.get(opcode, 0.0) + latency_us
        self.total_instructions += 1

    def hot_ops(self):
        return [op for op, n in self.op_frequency.items() if n >= self.hot_threshold]


def jit_dce(prog: Program) -> Program:
    """Drops NOPs and instructions whose result no later instruction reads (compiler.c:398-431)."""
    live, keep = set(), []
    for ins in reversed(prog.instructions):
        op = ins.opcode
        if op == Op.NOP:
            continue
        if op in (Op.STORE, Op.HALT, Op.BRANCH):
            keep.append(ins)
            if op in (Op.STORE, Op.BRANCH):
                live.add(ins.a)
            continue
        if ins.dest in live or not any(i.opcode == Op.STORE for i in prog.instructions):
            keep.append(ins)
            live.discard(ins.dest)
            if op != Op.LOAD:
                live.update((ins.a, ins.b))
                if op in (Op.ATTENTION, Op.FUSED_LINEAR):
                    live.add(ins.immediate if op == Op.ATTENTION else ins.shape_b[0])
    return prog.clone_with(reversed(keep))


def jit_fuse(prog: Program) -> Program:
    """MATMUL -> ADD (-> activation) chains become one FUSED_LINEAR whose epilogue carries bias and activation
    (compiler.c:255-319).  FUSED_LINEAR: dest, a = input, b = weight reg, shape_b[0] = bias reg, immediate = act op."""
    ins, out, i = prog.instructions, [], 0

    def reads(reg, start):
        return sum(1 for x in ins[start:] if x.opcode not in (Op.LOAD, Op.HALT, Op.NOP) and reg in (x.a, x.b))

    while i < len(ins):
        m = ins[i]
        if m.opcode == Op.MATMUL and i + 1 < len(ins) and ins[i + 1].opcode == Op.ADD and ins[i + 1].a == m.dest \
                and reads(m.dest, i + 1) == 1:
            add = ins[i + 1]
            act, dest, step = 0, add.dest, 2
            if i + 2 < len(ins) and ins[i + 2].opcode in (Op.RELU, Op.GELU, Op.SILU) and ins[i + 2].a == add.dest \
                    and reads(add.dest, i + 2) == 1:
                act, dest, step = int(ins[i + 2].opcode), ins[i + 2].dest, 3
            out.append(Instruction(Op.FUSED_LINEAR, dest, m.a, m.b, act, shape_b=(add.b, 0)))
            i += step
        else:
            out.append(m)
            i += 1
    return prog.clone_with(out)


def jit_specialize(prog: Program, batch, seq_len, dim) -> Program:
    """Records the concrete shapes on MATMUL / ATTENTION instructions (compiler.c:220-253)."""
    out = []
    for ins in prog.instructions:
        if ins.opcode in (Op.MATMUL, Op.ATTENTION, Op.FUSED_LINEAR):
            ins = Instruction(ins.opcode, ins.dest, ins.a, ins.b, ins.immediate, (batch * seq_len, dim), ins.shape_b)
        out.append(ins)
    return prog.clone_with(out)


def jit_optimize(profile: Optional[JITProfile], prog: Program) -> Program:
    """Pass pipeline of jit_pipeline.c:31-54: fuse -> dead-code elimination."""
    return jit_dce(jit_fuse(prog))


class VM:
    """Register VM (vm.c).  ``run`` executes until HALT or the step limit; returns the value of the last STORE (or
    of the last written register)."""

    def __init__(self, cfg: NPEConfig = None):
        self.cfg = cfg or NPEConfig()
        self.program: Optional[Program] = None
        self.trace: List[Instruction] = []
        self.profile = JITProfile(self.cfg.jit_hot_threshold) if self.cfg.jit_enabled else None
        self.regs = [None] * NUM_REGS

    def load(self, prog: Program):
        if self.cfg.verification_mode:
            ok, msgs = verify_program(prog)
            if not ok:
                raise ValueError("; ".join(msgs))
        self.program = prog

    def optimize(self):
        self.program = jit_optimize(self.profile, self.program)
        return self.program

    def _load(self, ins):
        r, c = ins.shape_a
        n = r * c if c else r
        v = self.program.memory[ins.immediate: ins.immediate + n]
        return v.view(r, c) if c else v

    def run(self, x):
        prog, regs = self.program, self.regs
        regs[:] = [None] * NUM_REGS
        regs[0] = x
        pc, steps, result, last = 0, 0, None, x
        timed = self.profile is not None and not x.is_cuda
        while pc < len(prog.instructions):
            steps += 1
            if steps > self.cfg.step_limit:
                raise RuntimeError("NPE step limit exceeded")
            ins = prog.instructions[pc]
            op = ins.opcode
            t0 = time.perf_counter() if timed else 0.0
            if self.cfg.trace_execution:
                self.trace.append(ins)
            if op == Op.HALT:
                break
            if op == Op.BRANCH:
                cond = regs[ins.a]
                pc = ins.immediate if (cond is None or bool((cond > 0).any())) else pc + 1
                continue
            if op == Op.LOAD:
                val = self._load(ins)
            elif op == Op.STORE:
                result = regs[ins.a]
                val = None
            elif op == Op.MATMUL:
                w = regs[ins.b]
                val = ops.linear(regs[ins.a], w.T.to(regs[ins.a].dtype)) if w.dim() == 2 else regs[ins.a] * w
            elif op == Op.FUSED_LINEAR:
                xin = regs[ins.a]
                val = ops.linear(xin, regs[ins.b].T.to(xin.dtype), regs[ins.shape_b[0]].to(xin.dtype))
                if ins.immediate:
                    val = _UNARY[Op(ins.immediate)](val)
            elif op in _UNARY:
                val = _UNARY[op](regs[ins.a])
            elif op in _BINARY:
                val = _BINARY[op](regs[ins.a], regs[ins.b])
            elif op == Op.SOFTMAX:
                val = torch.softmax(regs[ins.a], dim=-1)
            elif op == Op.LAYERNORM:
                val = tnn.functional.layer_norm(regs[ins.a], regs[ins.a].shape[-1:])
            elif op == Op.ATTENTION:
                q, k, v = regs[ins.a], regs[ins.b], regs[ins.immediate]
                val = torch.softmax(q @ k.transpose(-1, -2) / q.shape[-1] ** 0.5, dim=-1) @ v
            elif op == Op.MSE:
                val = (regs[ins.a] - regs[ins.b]).pow(2).mean()
            elif op == Op.CROSSENTROPY:
                val = tnn.functional.cross_entropy(regs[ins.a], regs[ins.b].long())
            elif op == Op.CONCAT:
                val = torch.cat([regs[ins.a], regs[ins.b]], dim=-1)
            elif op == Op.SPLIT:
                val = regs[ins.a].chunk(2, dim=-1)[ins.immediate & 1]
            elif op == Op.DROPOUT:
                val = regs[ins.a]
            elif op == Op.EMBEDDING:
                val = regs[ins.b][regs[ins.a].long()]
            elif op == Op.NOP:
                val = None
            else:
                raise NotImplementedError(f"opcode {op}")
            if val is not None and op != Op.STORE:
                regs[ins.dest] = val
                last = val
            if timed:
                self.profile.record(int(op), (time.perf_counter() - t0) * 1e6)
            pc += 1
        return result if result is not None else last


    # ---- single-launch interpreter (csrc/npe_interp.cu; the host library runs the same instruction code on CPU)
    def _encoded(self):
        import numpy as np
        rows = [[int(i.opcode), i.dest, i.a, i.b, i.immediate, i.shape_a[0], i.shape_a[1], i.shape_b[0]] for i in self.program.instructions]
        return np.ascontiguousarray(np.array(rows, dtype=np.int32).reshape(len(rows), 8))

    def plan_rows(self, in_width: int):
        """(code, widest register, output width) from the interpreter's planner; code 0 means the program can run
        there, -3 that it uses an instruction the interpreter leaves to ``run`` (ATTENTION, BRANCH, ...)."""
        import ctypes as C
        from .. import _build
        L = _build.load_host()
        prog = self._encoded()
        maxw, out_w = C.c_int(0), C.c_int(0)
        rc = L.sx_oracle_npe_plan(C.c_void_p(prog.ctypes.data), C.c_int(len(prog)), C.c_longlong(self.program.memory.numel()),
                                  C.c_int(in_width), C.byref(maxw), C.byref(out_w))
        return rc, maxw.value, out_w.value

    def run_rows(self, x: torch.Tensor) -> torch.Tensor:
        """The whole program in one call per batch: every row of x [..., width] goes through the interpreter with its
        registers on chip. Inference only (no autograd). Raises NotImplementedError for programs the planner refuses
        with -3 and ValueError for malformed ones."""
        import ctypes as C
        from .. import _build
        from ..ops import _lib
        width = x.shape[-1]
        rc, _, out_w = self.plan_rows(width)
        if rc == -3:
            raise NotImplementedError("program uses instructions outside the row interpreter")
        if rc != 0:
            raise ValueError(f"program does not pass the interpreter's planner (code {rc})")
        prog = self._encoded()
        xf = x.detach().reshape(-1, width).float().contiguous()
        mem = self.program.memory.detach().to(x.device).float().contiguous()     # the kernel dereferences it on x's device
        out = torch.empty(xf.shape[0], out_w, dtype=torch.float32, device=x.device)
        if x.is_cuda:
            dev_prog = torch.from_numpy(prog).to(x.device)
            _lib.call("sx_npe_run", C.c_void_p(prog.ctypes.data), _lib.ptr(dev_prog), C.c_int(len(prog)), _lib.ptr(mem),
                      C.c_longlong(mem.numel()), _lib.ptr(xf), C.c_longlong(xf.shape[0]), C.c_int(width), _lib.ptr(out),
                      C.c_int(out_w), _lib.stream())
        else:
            L = _build.load_host()
            rc = L.sx_oracle_npe_run(C.c_void_p(prog.ctypes.data), C.c_int(len(prog)), C.c_void_p(mem.data_ptr()), C.c_longlong(mem.numel()),
                                     C.c_void_p(xf.data_ptr()), C.c_longlong(xf.shape[0]), C.c_int(width), C.c_void_p(out.data_ptr()),
                                     C.c_int(out_w))
            if rc != 0:
                raise RuntimeError(f"interpreter failed with code {rc}")
        return out.reshape(*x.shape[:-1], out_w).to(x.dtype)


class NPELayer(Module):
    """A compiled program as an ``nn`` module: parameters are the program memory; the fused program is built once."""

    def __init__(self, dim, hidden=None, kind="mlp", seq_len=0, cfg: NPEConfig = None, device=None):
        super().__init__()
        self.program = compile_mlp(dim, hidden or 4 * dim, device=device) if kind == "mlp" else \
            compile_attention(seq_len, dim, device=device)
        self.vm = VM(cfg)
        self.vm.load(self.program)
        if self.vm.cfg.jit_enabled:
            self.vm.optimize()

    def forward(self, x):
        return self.vm.run(x)


NPEModel = NPELayer
NPEProgram = Program
NPEVM = VM
