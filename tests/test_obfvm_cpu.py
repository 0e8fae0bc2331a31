"""Native-logic obfuscation: flattened control flow and the per-program bytecode must compute what the plain IR
computes; the static graph becomes a star; tampering is caught by validation; sealed strings; debugger signals."""
import pytest

from sneppx_alg_b200.security.obfuscation import ObfuscatedRoutine, StringVault, debugger_signals

COLLATZ = """
entry: movi r1 0 ; jmp loop
loop:  cmpi r0 1 ; jle done step
step:  mov r2 r0 ; movi r3 1 ; and r2 r3 ; cmpi r2 0 ; jz even odd
even:  mov r4 r0 ; movi r5 0 ; jmp halve
halve: cmpi r4 2 ; jle halved sub2
sub2:  addi r4 -2 ; addi r5 1 ; jmp halve
halved: cmpi r4 2 ; jz plus1 set
plus1: addi r5 1 ; jmp set
set:   mov r0 r5 ; addi r1 1 ; out r0 ; jmp loop
odd:   mov r6 r0 ; add r0 r6 ; add r0 r6 ; addi r0 1 ; addi r1 1 ; out r0 ; jmp loop
done:  ret r1
"""


def collatz(n):
    steps, seq = 0, []
    while n > 1:
        n = n // 2 if n % 2 == 0 else 3 * n + 1
        steps += 1
        seq.append(n)
    return steps, seq


def test_flattening_and_bytecode_preserve_behaviour():
    for n in (1, 6, 7, 12):
        plain = ObfuscatedRoutine(COLLATZ)
        want = collatz(n)
        assert plain.run_ir(n) == want
        assert plain.compile(seed=1).run(n) == want
        flat = ObfuscatedRoutine(COLLATZ).flatten(seed=42)
        assert flat.run_ir(n) == want and flat.compile(seed=7).run(n) == want
        plain.close()
        flat.close()


def test_flattened_graph_is_a_star_and_encodings_differ():
    plain, flat = ObfuscatedRoutine(COLLATZ), ObfuscatedRoutine(COLLATZ).flatten(seed=3)
    nb = plain.num_blocks
    assert any(len(plain.successors(b)) == 2 and 1 not in plain.successors(b) for b in range(nb))
    real = range(2, 2 + nb)                       # after flattening: prologue, dispatcher, the shuffled real blocks
    assert flat.num_blocks > 2 * nb
    assert all(flat.successors(b) in ([1], []) for b in real)      # every real block only returns to the dispatcher
    a = ObfuscatedRoutine(COLLATZ).compile(seed=1)
    b = ObfuscatedRoutine(COLLATZ).compile(seed=2)
    ba, bb = a.bytecode(), b.bytecode()
    assert len(ba) == len(bb) and ba != bb and sum(x != y for x, y in zip(ba, bb)) > len(ba) // 4
    # equal instructions at different positions encode differently (the opcode byte depends on the position)
    ops = {ba[i] for i in range(0, len(ba), 8)}
    assert len(ops) > 12


def test_validation_catches_tampering_and_limits():
    r = ObfuscatedRoutine("entry: movi r0 5 ; jmp next\nnext: addi r0 1 ; ret r0").compile(seed=5)
    assert r.run() == (6, []) and r.validate() == 0
    size = len(r.bytecode())
    r.poke(12, 0xFF)                              # the jump target now points far outside the program
    r.poke(13, 0xFF)
    assert r.validate() == -4
    with pytest.raises(RuntimeError, match="jump target"):
        r.run()
    spin = ObfuscatedRoutine("entry: jmp entry").compile()
    with pytest.raises(RuntimeError, match="step limit"):
        spin.run(step_limit=1000)
    with pytest.raises(ValueError, match="unknown label"):
        ObfuscatedRoutine("entry: jmp nowhere")
    with pytest.raises(ValueError, match="does not end"):
        ObfuscatedRoutine("entry: movi r0 1")
    with pytest.raises(ValueError, match="reserved"):
        ObfuscatedRoutine("entry: movi r15 1 ; ret r15")
    assert size % 8 == 0


def test_string_vault_and_debugger_signals():
    v = StringVault(bytes(range(32)))
    sealed = v.seal("db_password", "correct horse battery staple")
    assert b"horse" not in sealed and len(sealed) == 28
    assert v.seal("other", "correct horse battery staple") != sealed          # the id is part of the keystream
    opened = v.open("db_password")
    with opened as s:
        assert s == "correct horse battery staple"
    assert opened.wiped
    sig = debugger_signals()
    assert set(sig) == {"tracer_attached", "ld_preload", "timing_anomaly"} and sig["tracer_attached"] is False
