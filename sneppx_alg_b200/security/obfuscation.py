"""S2 obfuscation pipeline for NPE bytecode programs: instruction substitution, opaque-predicate dead code, NOP
padding, and sealing of the serialized program (code + weights) under an authenticated cipher.

The reference's S2 layer (``security/obfuscation/*.cpp``: instruction substitution, opaque predicates, control-flow
changes, string encryption, pipeline driver) transforms code; the code this framework ships to untrusted hosts is NPE
bytecode, so the passes work on ``algorithms.npe.Program``. Every pass preserves the program's result exactly up to
floating-point reassociation (substitutions use only sign flips and doubled negations, which are exact), keeps branch
targets consistent when instructions move, and leaves a program that still passes ``verify_program``.
"""
from __future__ import annotations

import json
import os
import random
import struct
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch

from ..algorithms.npe import NUM_REGS, Instruction, Op, Program, verify_program
from . import crypto


@dataclass
class ObfuscationConfig:
    substitute: bool = True
    opaque_predicates: int = 2
    nop_padding: float = 0.2
    seed: int = 0


def _free_registers(prog: Program) -> List[int]:
    used = {0}
    for ins in prog.instructions:
        used.update((ins.dest, ins.a, ins.b))
        if ins.opcode == Op.ATTENTION:
            used.add(ins.immediate)
        if ins.opcode == Op.FUSED_LINEAR:
            used.add(ins.shape_b[0])
    return [r for r in range(1, NUM_REGS) if r not in used]


def _rebuild(prog: Program, groups: List[List[Instruction]]) -> Program:
    """`groups[i]` replaces original instruction i; branch targets are remapped to the first instruction of the
    group that replaces their old target."""
    start, pc = [], 0
    for g in groups:
        start.append(pc)
        pc += len(g)
    out = []
    for i, g in enumerate(groups):
        for ins in g:
            if ins.opcode == Op.BRANCH and getattr(ins, "_orig_target", None) is not None:
                ins = Instruction(ins.opcode, ins.dest, ins.a, ins.b, start[ins._orig_target], ins.shape_a, ins.shape_b)
            out.append(ins)
    p = prog.clone_with(out)
    p.max_instructions = max(prog.max_instructions, len(out) + 8)
    return p


def _tag_branches(prog: Program) -> List[Instruction]:
    tagged = []
    for ins in prog.instructions:
        c = Instruction(ins.opcode, ins.dest, ins.a, ins.b, ins.immediate, ins.shape_a, ins.shape_b)
        c._orig_target = ins.immediate if ins.opcode == Op.BRANCH else None
        tagged.append(c)
    return tagged


def substitute_instructions(prog: Program, seed: int = 0) -> Program:
    """SUB a, b -> NEG t, b ; ADD a, t.   ADD a, b -> NEG t, b ; SUB a, t.   Unary f(x) -> NEG t ; NEG t ; f(t) for a
    random subset (needs one free register; returns the program unchanged when there is none)."""
    free = _free_registers(prog)
    if not free:
        return prog
    t = free[0]
    rng = random.Random(seed)
    groups = []
    for ins in _tag_branches(prog):
        if ins.opcode == Op.SUB:
            groups.append([Instruction(Op.NEG, t, ins.b), Instruction(Op.ADD, ins.dest, ins.a, t)])
        elif ins.opcode == Op.ADD and rng.random() < 0.7:
            groups.append([Instruction(Op.NEG, t, ins.b), Instruction(Op.SUB, ins.dest, ins.a, t)])
        elif ins.opcode in (Op.RELU, Op.TANH, Op.SIGMOID, Op.GELU, Op.SILU) and rng.random() < 0.7:
            groups.append([Instruction(Op.NEG, t, ins.a), Instruction(Op.NEG, t, t), Instruction(ins.opcode, ins.dest, t)])
        else:
            groups.append([ins])
    return _rebuild(prog, groups)


def insert_opaque_predicates(prog: Program, count: int = 2, seed: int = 0) -> Program:
    """Before `count` random instructions: t = EXP(r0) (always positive), BRANCH on t over a block of junk arithmetic
    that is never executed. Needs two free registers."""
    free = _free_registers(prog)
    n = len(prog.instructions)
    if len(free) < 2 or n < 2 or count <= 0:
        return prog
    t, junk = free[0], free[1]
    rng = random.Random(seed)
    sites = set(rng.sample(range(1, n), min(count, n - 1)))
    groups = []
    for i, ins in enumerate(_tag_branches(prog)):
        if i in sites:
            br = Instruction(Op.BRANCH, 0, t, 0, 0)
            br._orig_target = i          # jumps to the start of this group's real instruction, fixed up below
            block = [Instruction(Op.EXP, t, 0), br, Instruction(Op.SIN, junk, 0), Instruction(Op.MUL, junk, junk, junk),
                     Instruction(Op.STORE, a=junk, immediate=0), ins]
            groups.append(block)
        else:
            groups.append([ins])
    p = _rebuild(prog, groups)
    # the opaque branches must land on the real instruction of their own group, which sits 4 slots after the branch
    fixed = []
    for pc, ins in enumerate(p.instructions):
        if ins.opcode == Op.BRANCH and ins.a == t:
            ins = Instruction(Op.BRANCH, 0, t, 0, pc + 4)
        fixed.append(ins)
    return p.clone_with(fixed)


def pad_with_nops(prog: Program, ratio: float = 0.2, seed: int = 0) -> Program:
    rng = random.Random(seed)
    groups = [[Instruction(Op.NOP), ins] if rng.random() < ratio else [ins] for ins in _tag_branches(prog)]
    return _rebuild(prog, groups)


class ObfuscationPipeline:
    """Runs the configured passes in order and checks the result with the bytecode verifier."""

    def __init__(self, config: Optional[ObfuscationConfig] = None):
        self.config = config or ObfuscationConfig()
        self.passes: List[Callable[[Program], Program]] = []
        c = self.config
        if c.substitute:
            self.passes.append(lambda p: substitute_instructions(p, c.seed))
        if c.opaque_predicates:
            self.passes.append(lambda p: insert_opaque_predicates(p, c.opaque_predicates, c.seed + 1))
        if c.nop_padding:
            self.passes.append(lambda p: pad_with_nops(p, c.nop_padding, c.seed + 2))

    def run(self, prog: Program) -> Program:
        limit = prog.max_instructions
        for f in self.passes:
            prog = f(prog)
        prog.max_instructions = max(limit, len(prog.instructions) + 8)
        ok, msgs = verify_program(prog)
        if not ok:
            raise RuntimeError("obfuscated program fails verification: " + "; ".join(msgs))
        return prog


# ----------------------------------------------------------------------------------------- sealing
def serialize_program(prog: Program) -> bytes:
    code = [[int(i.opcode), i.dest, i.a, i.b, i.immediate, list(i.shape_a), list(i.shape_b)] for i in prog.instructions]
    head = json.dumps({"code": code, "max": prog.max_instructions, "mem": prog.memory.numel()}).encode()
    return struct.pack("<I", len(head)) + head + prog.memory.detach().float().cpu().numpy().tobytes()


def deserialize_program(blob: bytes) -> Program:
    (n,) = struct.unpack("<I", blob[:4])
    head = json.loads(blob[4:4 + n])
    p = Program(head["mem"], head["max"])
    with torch.no_grad():
        p.memory.copy_(torch.frombuffer(bytearray(blob[4 + n:]), dtype=torch.float32))
    p.instructions = [Instruction(c[0], c[1], c[2], c[3], c[4], tuple(c[5]), tuple(c[6])) for c in head["code"]]
    return p


def seal_program(prog: Program, key: bytes) -> bytes:
    """nonce || ChaCha20-Poly1305(serialized program): code and weights are unreadable and tamper-evident at rest."""
    nonce = os.urandom(12)
    return nonce + crypto.aead_encrypt(key, nonce, serialize_program(prog), b"sneppx-npe")


def unseal_program(blob: bytes, key: bytes) -> Program:
    return deserialize_program(crypto.aead_decrypt(key, blob[:12], blob[12:], b"sneppx-npe"))
