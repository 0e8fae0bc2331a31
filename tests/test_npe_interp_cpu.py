"""The row interpreter for NPE bytecode (instruction code shared with the CUDA kernel) against the host VM."""
import pytest
import torch

from sneppx_alg_b200.algorithms import npe
from sneppx_alg_b200.algorithms.npe import Instruction, Op, Program


def _vm(prog, jit=False):
    vm = npe.VM(npe.NPEConfig(jit_enabled=jit))
    vm.load(prog)
    return vm


def test_compiled_mlp_fused_and_unfused():
    torch.manual_seed(0)
    prog = npe.compile_mlp(24, 40)
    with torch.no_grad():
        prog.memory.normal_(0, 0.3)
    x = torch.randn(3, 5, 24)
    vm = _vm(prog)
    want = vm.run(x)
    got = vm.run_rows(x)
    assert got.shape == want.shape and torch.allclose(got, want, atol=1e-5)
    fused = npe.VM(npe.NPEConfig())
    fused.load(prog)
    fused.optimize()
    assert any(i.opcode == Op.FUSED_LINEAR for i in fused.program.instructions)
    assert torch.allclose(fused.run_rows(x), want, atol=1e-5)
    rc, maxw, out_w = fused.plan_rows(24)
    assert (rc, maxw, out_w) == (0, 40, 24)


def _program(instructions, memory):
    p = Program(len(memory), 64)
    with torch.no_grad():
        p.memory.copy_(torch.tensor(memory))
    p.instructions = instructions
    return p


def test_every_supported_instruction_matches_the_vm():
    torch.manual_seed(1)
    D = 8
    mem = torch.randn(D * 6 + D + 6).tolist()
    W, bias = 0, D * 6                                     # W [8, 6] at 0, vector [8] at 48, vector [6] at 56
    ins = [
        Instruction(Op.LOAD, 1, immediate=W, shape_a=(D, 6)),
        Instruction(Op.LOAD, 2, immediate=bias, shape_a=(D, 0)),
        Instruction(Op.LOAD, 9, immediate=bias + D, shape_a=(6, 0)),
        Instruction(Op.ADD, 3, 0, 2), Instruction(Op.SUB, 3, 3, 0), Instruction(Op.MUL, 3, 3, 0), Instruction(Op.TANH, 3, 3),
        Instruction(Op.LAYERNORM, 4, 3), Instruction(Op.SIGMOID, 5, 4), Instruction(Op.DIV, 5, 4, 5),
        Instruction(Op.MATMUL, 6, 5, 1),                    # [8] x [8, 6] -> [6]
        Instruction(Op.MATMUL, 6, 6, 9),                    # vector operand: elementwise product
        Instruction(Op.SOFTMAX, 7, 6), Instruction(Op.CONCAT, 8, 7, 6), Instruction(Op.SPLIT, 10, 8, immediate=1),
        Instruction(Op.EXP, 11, 10), Instruction(Op.SQRT, 11, 11), Instruction(Op.LOG, 11, 11), Instruction(Op.NEG, 11, 11),
        Instruction(Op.SIN, 12, 11), Instruction(Op.COS, 13, 11), Instruction(Op.ADD, 12, 12, 13), Instruction(Op.GELU, 12, 12),
        Instruction(Op.SILU, 12, 12), Instruction(Op.RELU, 13, 12), Instruction(Op.DROPOUT, 13, 13), Instruction(Op.NOP),
        Instruction(Op.STORE, a=8),                         # the [12] concat is the result ...
        Instruction(Op.NEG, 8, 8),                          # ... even though its register changes afterwards
        Instruction(Op.HALT), Instruction(Op.EXP, 8, 8),
    ]
    prog = _program(ins, mem)
    vm = npe.VM(npe.NPEConfig(jit_enabled=False, verification_mode=0))
    vm.load(prog)
    x = torch.randn(7, D)
    want, got = vm.run(x), vm.run_rows(x)
    assert want.shape == (7, 12) and torch.allclose(got, want, atol=1e-5)
    # without a STORE the last written register is the result
    prog2 = _program(ins[:13], mem)
    vm.load(prog2)
    assert torch.allclose(vm.run_rows(x), vm.run(x), atol=1e-5)


def test_planner_refuses_what_it_cannot_run():
    vm = npe.VM(npe.NPEConfig(jit_enabled=False, verification_mode=0))
    vm.load(npe.compile_attention(4, 8))
    assert vm.plan_rows(8)[0] == -3
    with pytest.raises(NotImplementedError):
        vm.run_rows(torch.randn(4, 8))
    vm.load(_program([Instruction(Op.BRANCH, 0, 0, 0, 0)], [0.0]))
    assert vm.plan_rows(4)[0] == -3
    vm.load(_program([Instruction(Op.LOAD, 1, immediate=2, shape_a=(4, 4))], [0.0] * 8))       # matrix past the end of memory
    assert vm.plan_rows(4)[0] == -2
    vm.load(_program([Instruction(Op.LOAD, 1, immediate=0, shape_a=(3, 0)), Instruction(Op.ADD, 2, 0, 1)], [0.0] * 8))
    with pytest.raises(ValueError):
        vm.run_rows(torch.randn(2, 4))                                                          # widths 4 and 3
    vm.load(_program([Instruction(Op.ADD, 99, 0, 0)], [0.0]))
    assert vm.plan_rows(4)[0] == -1
