"""NPE bytecode obfuscation: every pass keeps the program's result, the pipeline output passes the verifier, sealed
programs round-trip and reject tampering."""
import os

import pytest
import torch

from sneppx_alg_b200.algorithms.npe import VM, Instruction, NPEConfig, Op, Program, compile_attention, compile_mlp
from sneppx_alg_b200.security import obfuscation as ob


def _run(prog, x):
    vm = VM(NPEConfig(jit_enabled=False))
    vm.load(prog)
    return vm.run(x)


@pytest.mark.parametrize("make,x", [(lambda: compile_mlp(8, 16, seed=1), torch.randn(4, 8)),
                                    (lambda: compile_attention(6, 8, seed=2), torch.randn(6, 8))])
def test_passes_preserve_results(make, x):
    prog = make()
    want = _run(prog, x)
    for f in (lambda p: ob.substitute_instructions(p, 3), lambda p: ob.insert_opaque_predicates(p, 3, 4), lambda p: ob.pad_with_nops(p, 0.5, 5)):
        got = _run(f(prog), x)
        assert torch.allclose(got, want, atol=1e-6)
    out = ob.ObfuscationPipeline(ob.ObfuscationConfig(opaque_predicates=3, nop_padding=0.4, seed=7)).run(prog)
    assert len(out.instructions) > len(prog.instructions) + 6
    assert torch.allclose(_run(out, x), want, atol=1e-6)
    ops_used = {int(i.opcode) for i in out.instructions}
    assert int(Op.BRANCH) in ops_used and int(Op.NOP) in ops_used
    has_arith = any(i.opcode in (Op.ADD, Op.SUB, Op.RELU) for i in prog.instructions)
    assert (int(Op.NEG) in ops_used) == has_arith   # substitutions only where there is arithmetic to rewrite


def test_branch_targets_follow_moved_instructions():
    p = Program(4, 32)
    I = Instruction  # noqa: E741
    # r1 = exp(x) (positive) -> branch over the instruction that would negate the input
    for ins in (I(Op.EXP, 1, 0), I(Op.BRANCH, 0, 1, 0, 3), I(Op.NEG, 0, 0), I(Op.TANH, 2, 0), I(Op.SUB, 3, 2, 0), I(Op.STORE, a=3, immediate=0), I(Op.HALT)):
        p.append(ins)
    x = torch.randn(5)
    want = torch.tanh(x) - x
    assert torch.allclose(_run(p, x), want)
    out = ob.ObfuscationPipeline(ob.ObfuscationConfig(opaque_predicates=4, nop_padding=0.6, seed=11)).run(p)
    assert torch.allclose(_run(out, x), want, atol=1e-6)


def test_sealed_program_roundtrip_and_tamper():
    prog = compile_mlp(8, 16, seed=3)
    key = os.urandom(32)
    blob = ob.seal_program(prog, key)
    back = ob.unseal_program(blob, key)
    x = torch.randn(2, 8)
    assert torch.equal(_run(back, x), _run(prog, x)) and len(back.instructions) == len(prog.instructions)
    assert prog.memory.detach().numpy().tobytes() not in blob           # weights are not readable at rest
    bad = bytearray(blob)
    bad[40] ^= 1
    with pytest.raises(ValueError):
        ob.unseal_program(bytes(bad), key)
    with pytest.raises(ValueError):
        ob.unseal_program(blob, os.urandom(32))
