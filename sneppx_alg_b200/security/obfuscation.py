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


# ----------------------------------------------------------------------------------------------- native-logic obfuscation
class ObfuscatedRoutine:
    """A routine written in the small register IR of ``csrc/host/obfvm.cpp`` ("label: movi r0 5 ; cmpi r0 3 ;
    jg big small"), optionally control-flow flattened, compiled to a bytecode whose opcode encoding is private to
    this compilation, and run by the native virtual machine. The reference's passes of the same purpose:
    security/obfuscation/cfg_flatten.cpp, security/obfuscation/vm.cpp."""

    def __init__(self, source: str):
        import ctypes as C
        L = self._lib()
        self._C, self._g = C, L.sx_obf_parse(source.encode())
        err = L.sx_obf_cfg_error(self._g).decode()
        if err:
            L.sx_obf_cfg_free(self._g)
            self._g = None
            raise ValueError(err)
        self._p = None

    @staticmethod
    def _lib():
        import ctypes as C

        from .. import _build
        L = _build.load_host()
        if not getattr(L, "_obf_ready", False):
            L.sx_obf_parse.restype = L.sx_obf_compile.restype = C.c_void_p
            L.sx_obf_parse.argtypes = [C.c_char_p]
            L.sx_obf_cfg_error.restype = C.c_char_p
            for f in ("sx_obf_cfg_error", "sx_obf_cfg_free", "sx_obf_cfg_blocks", "sx_obf_program_free", "sx_obf_program_size",
                      "sx_obf_validate"):
                getattr(L, f).argtypes = [C.c_void_p]
            L.sx_obf_program_size.restype = C.c_longlong
            L.sx_obf_cfg_successors.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
            L.sx_obf_flatten.argtypes = L.sx_obf_compile.argtypes = [C.c_void_p, C.c_ulonglong]
            L.sx_obf_flatten.restype = None
            sig = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_longlong]
            L.sx_obf_run_ir.argtypes = L.sx_obf_execute.argtypes = sig
            L.sx_obf_program_bytes.argtypes = [C.c_void_p, C.c_void_p]
            L.sx_obf_program_poke.argtypes = [C.c_void_p, C.c_longlong, C.c_ubyte]
            L.sx_obf_string_xform.argtypes = [C.c_char_p, C.c_ulonglong, C.c_char_p, C.c_void_p, C.c_size_t]
            L.sx_obf_string_xform.restype = None
            L.sx_obf_wipe.argtypes = [C.c_void_p, C.c_size_t]
            L.sx_obf_debugger_signals.argtypes = [C.c_double]
            L._obf_ready = True
        return L

    @property
    def num_blocks(self) -> int:
        return self._lib().sx_obf_cfg_blocks(self._g)

    def successors(self, block: int) -> List[int]:
        out = (self._C.c_int * 4)()
        n = self._lib().sx_obf_cfg_successors(self._g, block, out, 4)
        return [int(out[i]) for i in range(max(n, 0))]

    def flatten(self, seed: int = 0) -> "ObfuscatedRoutine":
        self._lib().sx_obf_flatten(self._g, seed)
        return self

    def compile(self, seed: int = 0) -> "ObfuscatedRoutine":
        if self._p:
            self._lib().sx_obf_program_free(self._p)
        self._p = self._lib().sx_obf_compile(self._g, seed)
        if not self._p:
            raise ValueError("program has an immediate outside 32 bits")
        return self

    def _run(self, fn, handle, args, step_limit):
        C = self._C
        a = (C.c_longlong * max(len(args), 1))(*args)
        out = (C.c_longlong * 256)()
        n_out, ret = C.c_int(0), C.c_longlong(0)
        rc = fn(handle, a, len(args), out, 256, C.byref(n_out), C.byref(ret), step_limit)
        if rc != 0:
            raise RuntimeError({-1: "undecodable opcode", -2: "step limit exceeded", -3: "register out of range",
                                -4: "jump target out of range", -5: "truncated program", -6: "ran off the end"}.get(rc, f"error {rc}"))
        return int(ret.value), [int(out[i]) for i in range(n_out.value)]

    def run_ir(self, *args, step_limit: int = 1_000_000):
        """Interpret the control-flow graph directly: (return value, values passed to ``out``)."""
        return self._run(self._lib().sx_obf_run_ir, self._g, args, step_limit)

    def run(self, *args, step_limit: int = 1_000_000):
        """Run the compiled bytecode on the virtual machine."""
        if not self._p:
            self.compile()
        return self._run(self._lib().sx_obf_execute, self._p, args, step_limit)

    def bytecode(self) -> bytes:
        n = self._lib().sx_obf_program_size(self._p)
        buf = self._C.create_string_buffer(n)
        self._lib().sx_obf_program_bytes(self._p, buf)
        return buf.raw

    def poke(self, offset: int, value: int) -> None:
        self._lib().sx_obf_program_poke(self._p, offset, value)

    def validate(self) -> int:
        return self._lib().sx_obf_validate(self._p)

    def close(self) -> None:
        L = self._lib()
        if self._p:
            L.sx_obf_program_free(self._p)
            self._p = None
        if self._g:
            L.sx_obf_cfg_free(self._g)
            self._g = None


class StringVault:
    """String literals kept sealed (ChaCha20 under a vault key and the string's id) and opened one at a time into a
    buffer that is wiped when the ``with`` block ends (security/obfuscation/string_encrypt.cpp)."""

    def __init__(self, key32: bytes):
        assert len(key32) == 32
        self._key, self._items = key32, {}

    def seal(self, name: str, text: str) -> bytes:
        import ctypes as C
        raw = text.encode()
        sid = int.from_bytes(hashlib_sha(name)[:8], "little")
        out = C.create_string_buffer(len(raw))
        ObfuscatedRoutine._lib().sx_obf_string_xform(self._key, sid, raw, out, len(raw))
        self._items[name] = out.raw
        return out.raw

    def open(self, name: str):
        import ctypes as C
        sealed = self._items[name]
        sid = int.from_bytes(hashlib_sha(name)[:8], "little")
        buf = C.create_string_buffer(len(sealed))
        ObfuscatedRoutine._lib().sx_obf_string_xform(self._key, sid, sealed, buf, len(sealed))
        return _OpenedString(buf)


def hashlib_sha(name: str) -> bytes:
    import hashlib
    return hashlib.sha256(name.encode()).digest()


class _OpenedString:
    def __init__(self, buf):
        self._buf = buf

    def __enter__(self):
        return self._buf.raw.decode()

    def __exit__(self, *exc):
        ObfuscatedRoutine._lib().sx_obf_wipe(self._buf, len(self._buf))

    @property
    def wiped(self) -> bool:
        return not any(self._buf.raw)


def debugger_signals(slow_factor: float = 50.0) -> dict:
    """Signs of being observed: an attached tracer, a preloaded library, a timing probe that ran ``slow_factor`` times
    slower than its own best (security/obfuscation/debug_detect.cpp)."""
    bits = ObfuscatedRoutine._lib().sx_obf_debugger_signals(slow_factor)
    return {"tracer_attached": bool(bits & 1), "ld_preload": bool(bits & 2), "timing_anomaly": bool(bits & 4)}
