"""S6 extensions: key custody and the operator-facing security surfaces.

* ``shamir_split`` / ``shamir_reconstruct``: k-of-n secret sharing over GF(2^8), byte by byte;
* ``KeyStore``: HSM-shaped store (keys live encrypted under a master key, are used by id, can be generated inside,
  wrapped under another key for transport and marked non-exportable);
* ``KeyCeremony``: a key is generated only once enough registered participants have approved, inside a time limit, and
  is handed out as Shamir shares; ``KeyRotationScheduler``: interval-based rotation with a rotate callback;
* ``PolicyDSL``: access rules (``allow|deny <subject> <action> <resource> [if <condition>]``) compiled to a small
  byte code and evaluated by a stack machine, first match wins, default deny;
* ``ThreatGraph`` (attack-path graph with DOT export), ``SecurityDashboard`` (named widgets, JSON / HTML snapshot),
  ``ComplianceReportBuilder`` (findings per control, text / JSON / single-page PDF output).

Reference behaviour: security/ui/s6_extensions.c (function families ``hsm_*``, ``shamir_*``, ``key_ceremony_*``,
``key_rotation_*``, ``policy_dsl_*``, ``threat_viz_*``, ``security_dashboard_*``, ``compliance_report*``). The key
vault and the hash-chained audit log themselves are in ``security/services.py``.
"""
from __future__ import annotations

import fnmatch
import html
import json
import os
import re
import struct
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from . import crypto

# ------------------------------------------------------------------------------------------------ GF(256) sharing
_EXP, _LOG = [0] * 512, [0] * 256


def _init_gf():
    x = 1
    for i in range(255):
        _EXP[i], _LOG[x] = x, i
        x ^= (x << 1) ^ (0x11B if x & 0x80 else 0)          # multiply by the generator 3 in the AES field
        x &= 0xFF
    for i in range(255, 512):
        _EXP[i] = _EXP[i - 255]


_init_gf()


def _gf_mul(a: int, b: int) -> int:
    return 0 if a == 0 or b == 0 else _EXP[_LOG[a] + _LOG[b]]


def _gf_div(a: int, b: int) -> int:
    if b == 0:
        raise ZeroDivisionError
    return 0 if a == 0 else _EXP[_LOG[a] + 255 - _LOG[b]]


def shamir_split(secret: bytes, n: int, k: int, rng: Callable[[int], bytes] = os.urandom) -> List[bytes]:
    """``n`` shares of which any ``k`` rebuild ``secret``; fewer than ``k`` carry no information about it. A share is
    one byte of x-coordinate (1..n) followed by one byte per secret byte."""
    if not 1 <= k <= n <= 255:
        raise ValueError("need 1 <= k <= n <= 255")
    coeffs = [bytes([s]) + rng(k - 1) for s in secret]       # per byte: a random polynomial with the secret at x = 0
    shares = []
    for x in range(1, n + 1):
        ys = bytearray()
        for c in coeffs:
            y = 0
            for a in reversed(c):                             # Horner
                y = _gf_mul(y, x) ^ a
            ys.append(y)
        shares.append(bytes([x]) + bytes(ys))
    return shares


def shamir_reconstruct(shares: Sequence[bytes]) -> bytes:
    """Lagrange interpolation at x = 0 over the given shares (give exactly the threshold number, or more)."""
    if not shares:
        raise ValueError("no shares")
    xs = [s[0] for s in shares]
    if len(set(xs)) != len(xs) or 0 in xs or len({len(s) for s in shares}) != 1:
        raise ValueError("shares must have distinct non-zero x and one length")
    out = bytearray()
    for i in range(1, len(shares[0])):
        acc = 0
        for j, sj in enumerate(shares):
            num = den = 1
            for m, xm in enumerate(xs):
                if m != j:
                    num, den = _gf_mul(num, xm), _gf_mul(den, xs[j] ^ xm)
            acc ^= _gf_mul(sj[i], _gf_div(num, den))
        out.append(acc)
    return bytes(out)


# ------------------------------------------------------------------------------------------------ key store
class KeyStoreError(RuntimeError):
    pass


@dataclass
class _KeyEntry:
    sealed: bytes
    kind: str
    exportable: bool
    created: float
    uses: int = 0


class KeyStore:
    """Keys addressed by id and kept sealed (ChaCha20-Poly1305 under the store's master key, key id as associated
    data) while at rest in the store. Operations take key ids; raw key bytes leave only through ``load_key`` of an
    exportable key or wrapped under another key of the store."""

    KINDS = {"aes256": 32, "chacha20": 32, "hmac": 32, "ed25519-seed": 32, "x25519": 32}

    def __init__(self, master_key: Optional[bytes] = None, capacity: int = 1024, clock: Callable[[], float] = time.time):
        self._master = master_key or os.urandom(32)
        if len(self._master) != 32:
            raise ValueError("the master key has 32 bytes")
        self.capacity, self.clock = capacity, clock
        self._keys: Dict[bytes, _KeyEntry] = {}

    def _seal(self, key_id: bytes, data: bytes) -> bytes:
        nonce = os.urandom(12)
        return nonce + crypto.aead_encrypt(self._master, nonce, data, key_id)

    def _open(self, key_id: bytes) -> bytes:
        e = self._keys.get(key_id)
        if e is None:
            raise KeyStoreError("no such key")
        e.uses += 1
        return crypto.aead_decrypt(self._master, e.sealed[:12], e.sealed[12:], key_id)

    def store_key(self, key_id: bytes, key_data: bytes, kind: str = "aes256", exportable: bool = True) -> None:
        if key_id in self._keys:
            raise KeyStoreError("key id already in use")
        if len(self._keys) >= self.capacity:
            raise KeyStoreError("key store is full")
        self._keys[key_id] = _KeyEntry(self._seal(key_id, key_data), kind, exportable, self.clock())

    def generate_key(self, kind: str = "aes256", key_id: Optional[bytes] = None, exportable: bool = False) -> bytes:
        if kind not in self.KINDS:
            raise KeyStoreError(f"unknown key type {kind!r}")
        key_id = key_id or os.urandom(8).hex().encode()
        self.store_key(key_id, os.urandom(self.KINDS[kind]), kind, exportable)
        return key_id

    def load_key(self, key_id: bytes) -> bytes:
        e = self._keys.get(key_id)
        if e is not None and not e.exportable:
            raise KeyStoreError("key is not exportable")
        return self._open(key_id)

    def delete_key(self, key_id: bytes) -> bool:
        return self._keys.pop(key_id, None) is not None

    def list_keys(self) -> List[bytes]:
        return sorted(self._keys)

    def key_count(self) -> int:
        return len(self._keys)

    def key_info(self, key_id: bytes) -> dict:
        e = self._keys.get(key_id)
        if e is None:
            raise KeyStoreError("no such key")
        return {"kind": e.kind, "exportable": e.exportable, "created": e.created, "uses": e.uses}

    # ---- use without export
    def mac(self, key_id: bytes, message: bytes) -> bytes:
        return crypto.hmac_sha256(self._open(key_id), message)

    def encrypt(self, key_id: bytes, plaintext: bytes, aad: bytes = b"") -> bytes:
        nonce = os.urandom(12)
        return nonce + crypto.aead_encrypt(self._open(key_id), nonce, plaintext, aad)

    def decrypt(self, key_id: bytes, sealed: bytes, aad: bytes = b"") -> bytes:
        return crypto.aead_decrypt(self._open(key_id), sealed[:12], sealed[12:], aad)

    def sign(self, key_id: bytes, message: bytes) -> bytes:
        if self._keys.get(key_id) is None or self._keys[key_id].kind != "ed25519-seed":
            raise KeyStoreError("not a signing key")
        return crypto.ed25519_sign(self._open(key_id), message)

    def public_key(self, key_id: bytes) -> bytes:
        e = self._keys.get(key_id)
        if e is None or e.kind not in ("ed25519-seed", "x25519"):
            raise KeyStoreError("not an asymmetric key")
        raw = self._open(key_id)
        return crypto.ed25519_public_key(raw) if e.kind == "ed25519-seed" else crypto.x25519(raw)

    # ---- transport
    def wrap_key(self, key_id: bytes, wrapping_key_id: bytes) -> bytes:
        """kind-length(1) || kind || nonce(12) || AEAD(key) under the wrapping key, key id as associated data."""
        e = self._keys.get(key_id)
        if e is None:
            raise KeyStoreError("no such key")
        kind = e.kind.encode()
        nonce = os.urandom(12)
        return bytes([len(kind)]) + kind + nonce + crypto.aead_encrypt(self._open(wrapping_key_id), nonce, self._open(key_id), key_id)

    def unwrap_key(self, wrapped: bytes, wrapping_key_id: bytes, key_id: bytes, exportable: bool = False) -> bytes:
        n = wrapped[0]
        kind, nonce, body = wrapped[1:1 + n].decode(), wrapped[1 + n:13 + n], wrapped[13 + n:]
        try:
            raw = crypto.aead_decrypt(self._open(wrapping_key_id), nonce, body, key_id)
        except ValueError as e:
            raise KeyStoreError("wrapped key does not authenticate") from e
        self.store_key(key_id, raw, kind, exportable)
        return key_id


# ------------------------------------------------------------------------------------------------ ceremony, rotation
class KeyCeremony:
    """Multi-party key generation. Participants are enrolled by a token (only its hash is kept); each approves with
    the token; ``execute`` succeeds once ``required`` distinct participants approved and the time limit has not run
    out, and returns (key id in the store, one Shamir share per approving participant, threshold = required)."""

    def __init__(self, participants: int, required: Optional[int] = None, timeout_s: float = 3600.0,
                 clock: Callable[[], float] = time.time):
        if participants < 1:
            raise ValueError("a ceremony needs participants")
        self.participants, self.required = participants, required or participants // 2 + 1
        if not 1 <= self.required <= participants:
            raise ValueError("required approvals out of range")
        self.timeout_s, self.clock = timeout_s, clock
        self._enrolled: Dict[bytes, str] = {}
        self._approved: List[str] = []
        self._started = clock()
        self.state = "open"                                   # open | executed | cancelled | expired

    def enroll(self, name: str, token: bytes) -> None:
        if len(self._enrolled) >= self.participants:
            raise ValueError("all participant seats are taken")
        self._enrolled[crypto.sha256(token)] = name

    def _check_open(self) -> bool:
        if self.state == "open" and self.clock() - self._started > self.timeout_s:
            self.state = "expired"
        return self.state == "open"

    def approve(self, token: bytes) -> bool:
        if not self._check_open():
            return False
        name = self._enrolled.get(crypto.sha256(token))
        if name is None or name in self._approved:
            return False
        self._approved.append(name)
        return True

    def status(self) -> dict:
        self._check_open()
        return {"state": self.state, "approved": len(self._approved), "present": len(self._enrolled), "required": self.required}

    def set_timeout(self, seconds: float) -> None:
        self.timeout_s = float(seconds)

    def cancel(self) -> bool:
        if self.state != "open":
            return False
        self.state = "cancelled"
        return True

    def execute(self, store: KeyStore, kind: str = "aes256", key_id: Optional[bytes] = None) -> Tuple[bytes, Dict[str, bytes]]:
        if not self._check_open():
            raise KeyStoreError(f"ceremony is {self.state}")
        if len(self._approved) < self.required:
            raise KeyStoreError(f"{len(self._approved)} of {self.required} approvals")
        kid = store.generate_key(kind, key_id, exportable=True)
        shares = shamir_split(store.load_key(kid), len(self._approved), self.required)
        store._keys[kid].exportable = False                   # from here on the key is used by id only
        self.state = "executed"
        return kid, dict(zip(self._approved, shares))


class KeyRotationScheduler:
    """Says when a key is due (``interval_s`` since the last rotation) and, with ``auto`` on, calls ``rotate`` from
    ``check``. ``rotate`` receives the rotation count and returns nothing."""

    def __init__(self, interval_s: float, rotate: Optional[Callable[[int], None]] = None, auto: bool = True,
                 clock: Callable[[], float] = time.time):
        if interval_s <= 0:
            raise ValueError("interval must be positive")
        self.interval_s, self.rotate, self.auto, self.clock = float(interval_s), rotate, auto, clock
        self.last, self.count = clock(), 0

    def remaining(self) -> float:
        return max(0.0, self.last + self.interval_s - self.clock())

    def check(self) -> bool:
        """True when a rotation is due; with ``auto`` it has been carried out by the time this returns."""
        if self.remaining() > 0:
            return False
        if self.auto:
            self.force_rotate()
        return True

    def force_rotate(self) -> int:
        self.count += 1
        self.last = self.clock()
        if self.rotate is not None:
            self.rotate(self.count)
        return self.count

    def set_auto(self, enabled: bool) -> None:
        self.auto = bool(enabled)


# ------------------------------------------------------------------------------------------------ policy language
# byte code: one opcode byte, then its operand. Strings and numbers are length-prefixed UTF-8 / 8-byte doubles.
OP_PUSH_ATTR, OP_PUSH_STR, OP_PUSH_NUM, OP_EQ, OP_NE, OP_LT, OP_LE, OP_GT, OP_GE, OP_IN, OP_MATCH, OP_AND, OP_OR, OP_NOT, \
    OP_GLOB, OP_RET_ALLOW, OP_RET_DENY, OP_JMP_FALSE = range(1, 19)
_CMP = {"==": OP_EQ, "!=": OP_NE, "<": OP_LT, "<=": OP_LE, ">": OP_GT, ">=": OP_GE, "in": OP_IN, "matches": OP_MATCH}
_TOKEN = re.compile(r'\s*(?:(\d+(?:\.\d+)?)|"((?:[^"\\]|\\.)*)"|(==|!=|<=|>=|<|>|\(|\))|([A-Za-z_][\w.]*))')


class PolicyError(ValueError):
    pass


class PolicyDSL:
    """Access rules, first match wins, default deny.

        allow role:admin * *
        allow role:ml-* deploy model/* if env == "staging" or (hour >= 8 and hour < 18)
        deny  * delete model/prod-* if not mfa

    A rule is ``allow|deny <subject glob> <action glob> <resource glob> [if <condition>]``. Conditions compare request
    attributes with literals (``== != < <= > >= in matches``), combine with ``and / or / not`` and parentheses; a bare
    attribute is its truth value. ``compile`` turns the rule list into byte code; ``evaluate`` runs it."""

    def __init__(self, rules: Iterable[str] = (), capacity: int = 512):
        self.capacity, self.rules = capacity, []
        for r in rules:
            self.add_rule(r)
        self._code: Optional[bytes] = None

    # ---- rule list
    def add_rule(self, rule: str) -> int:
        if len(self.rules) >= self.capacity:
            raise PolicyError("policy is full")
        self._parse(rule)
        self.rules.append(rule.strip())
        self._code = None
        return len(self.rules) - 1

    def set_rule(self, index: int, rule: str) -> None:
        self._parse(rule)
        self.rules[index] = rule.strip()
        self._code = None

    def remove_rule(self, index: int) -> bool:
        if not 0 <= index < len(self.rules):
            return False
        del self.rules[index]
        self._code = None
        return True

    def rule_count(self) -> int:
        return len(self.rules)

    def validate(self) -> List[str]:
        """Problems that do not stop compilation: rules that can never fire because an earlier unconditional rule
        with the same or a wider pattern decides first."""
        out, seen = [], []
        for i, r in enumerate(self.rules):
            eff, subj, act, res, cond = self._parse(r)
            for j, (s2, a2, r2) in seen:
                if all(fnmatch.fnmatchcase(x, y) for x, y in ((subj, s2), (act, a2), (res, r2))):
                    out.append(f"rule {i} is shadowed by rule {j}")
                    break
            if cond is None:
                seen.append((i, (subj, act, res)))
        return out

    # ---- parsing
    @staticmethod
    def _parse(rule: str):
        head, sep, cond = rule.strip().partition(" if ")
        parts = head.split()
        if len(parts) != 4 or parts[0] not in ("allow", "deny"):
            raise PolicyError(f"bad rule {rule!r}: want 'allow|deny subject action resource [if condition]'")
        if sep and not cond.strip():
            raise PolicyError(f"bad rule {rule!r}: empty condition")
        tokens = None
        if sep:
            tokens, pos = [], 0
            while pos < len(cond):
                if cond[pos:].strip() == "":
                    break
                m = _TOKEN.match(cond, pos)
                if not m:
                    raise PolicyError(f"bad condition near {cond[pos:]!r}")
                num, s, op, word = m.groups()
                tokens.append(("num", float(num)) if num is not None else ("str", re.sub(r"\\(.)", r"\1", s)) if s is not None
                              else ("op", op) if op is not None else ("word", word))
                pos = m.end()
            _CondCompiler(tokens).compile()               # syntax check
        return parts[0], parts[1], parts[2], parts[3], tokens

    # ---- compilation
    @staticmethod
    def _s(text: str) -> bytes:
        raw = text.encode()
        return struct.pack(">H", len(raw)) + raw

    def compile(self) -> bytes:
        code = bytearray()
        for r in self.rules:
            eff, subj, act, res, cond = self._parse(r)
            body = bytearray()
            for attr, pat in (("subject", subj), ("action", act), ("resource", res)):
                if pat != "*":
                    body += bytes([OP_PUSH_ATTR]) + self._s(attr) + bytes([OP_PUSH_STR]) + self._s(pat) + bytes([OP_GLOB])
                    body += bytes([OP_JMP_FALSE]) + b"\0\0"          # patched below: skip the rest of this rule
            if cond is not None:
                body += _CondCompiler(cond).compile() + bytes([OP_JMP_FALSE]) + b"\0\0"
            body += bytes([OP_RET_ALLOW if eff == "allow" else OP_RET_DENY])
            end, i = len(body), 0
            while i < end:                                   # point every rule-level jump at the rule's end
                op = body[i]
                if op in (OP_PUSH_ATTR, OP_PUSH_STR):
                    i += 3 + struct.unpack(">H", body[i + 1:i + 3])[0]
                elif op == OP_PUSH_NUM:
                    i += 9
                elif op == OP_JMP_FALSE:
                    body[i + 1:i + 3] = struct.pack(">H", end - (i + 3))
                    i += 3
                else:
                    i += 1
            code += body
        code.append(OP_RET_DENY)
        self._code = bytes(code)
        return self._code

    # ---- evaluation
    def evaluate(self, subject: str, action: str, resource: str, **attrs) -> bool:
        return self.run(self._code or self.compile(), {"subject": subject, "action": action, "resource": resource, **attrs})

    @staticmethod
    def run(code: bytes, request: Dict[str, Any], max_steps: int = 100000) -> bool:
        """The stack machine: returns True for allow. Unknown attributes read as None; comparing None is False."""
        stack: List[Any] = []
        pc = steps = 0
        while pc < len(code):
            steps += 1
            if steps > max_steps:
                raise PolicyError("policy program ran too long")
            op = code[pc]
            pc += 1
            if op in (OP_PUSH_ATTR, OP_PUSH_STR):
                n = struct.unpack(">H", code[pc:pc + 2])[0]
                text = code[pc + 2:pc + 2 + n].decode()
                pc += 2 + n
                stack.append(request.get(text) if op == OP_PUSH_ATTR else text)
            elif op == OP_PUSH_NUM:
                stack.append(struct.unpack(">d", code[pc:pc + 8])[0])
                pc += 8
            elif op == OP_NOT:
                stack.append(not stack.pop())
            elif op in (OP_AND, OP_OR):
                b, a = stack.pop(), stack.pop()
                stack.append(bool(a) and bool(b) if op == OP_AND else bool(a) or bool(b))
            elif op == OP_JMP_FALSE:
                off = struct.unpack(">H", code[pc:pc + 2])[0]
                pc += 2
                if not stack.pop():
                    pc += off
            elif op == OP_RET_ALLOW:
                return True
            elif op == OP_RET_DENY:
                return False
            else:
                b, a = stack.pop(), stack.pop()
                try:
                    if a is None:
                        v = False
                    elif op == OP_GLOB:
                        v = fnmatch.fnmatchcase(str(a), b)
                    elif op == OP_MATCH:
                        v = re.search(b, str(a)) is not None
                    elif op == OP_IN:
                        v = str(a) in [x.strip() for x in b.split(",")] if isinstance(b, str) else a in b
                    elif op == OP_EQ:
                        v = a == b
                    elif op == OP_NE:
                        v = a != b
                    else:
                        v = {OP_LT: a < b, OP_LE: a <= b, OP_GT: a > b, OP_GE: a >= b}[op]
                except TypeError:
                    v = False
                stack.append(v)
        return False


class _CondCompiler:
    """Recursive descent over condition tokens: or_expr := and_expr ('or' and_expr)*; and_expr := unary ('and' unary)*;
    unary := 'not' unary | '(' or_expr ')' | comparison; comparison := operand [cmp operand]."""

    def __init__(self, tokens):
        self.t, self.i = tokens, 0

    def _peek(self):
        return self.t[self.i] if self.i < len(self.t) else (None, None)

    def _take(self):
        tok = self._peek()
        self.i += 1
        return tok

    def compile(self) -> bytes:
        out = self._or()
        if self.i != len(self.t):
            raise PolicyError(f"unexpected {self._peek()[1]!r} in condition")
        return out

    def _or(self) -> bytes:
        out = self._and()
        while self._peek() == ("word", "or"):
            self._take()
            out += self._and() + bytes([OP_OR])
        return out

    def _and(self) -> bytes:
        out = self._unary()
        while self._peek() == ("word", "and"):
            self._take()
            out += self._unary() + bytes([OP_AND])
        return out

    def _unary(self) -> bytes:
        kind, v = self._peek()
        if (kind, v) == ("word", "not"):
            self._take()
            return self._unary() + bytes([OP_NOT])
        if (kind, v) == ("op", "("):
            self._take()
            out = self._or()
            if self._take() != ("op", ")"):
                raise PolicyError("missing ')'")
            return out
        left = self._operand()
        kind, v = self._peek()
        if (kind == "op" and v in _CMP) or (kind == "word" and v in ("in", "matches")):
            self._take()
            return left + self._operand() + bytes([_CMP[v]])
        return left

    def _operand(self) -> bytes:
        kind, v = self._take()
        if kind == "num":
            return bytes([OP_PUSH_NUM]) + struct.pack(">d", v)
        if kind == "str":
            return bytes([OP_PUSH_STR]) + PolicyDSL._s(v)
        if kind == "word" and v not in ("and", "or", "not", "in", "matches"):
            if v in ("true", "false"):
                return bytes([OP_PUSH_NUM]) + struct.pack(">d", 1.0 if v == "true" else 0.0)
            return bytes([OP_PUSH_ATTR]) + PolicyDSL._s(v)
        raise PolicyError(f"expected a value, found {v!r}")


# ------------------------------------------------------------------------------------------------ threat graph
class ThreatGraph:
    """Directed graph of "from this foothold an attacker reaches that asset by this technique". ``attack_paths`` lists
    the simple paths between two nodes, shortest first; ``export_dot`` writes Graphviz text."""

    def __init__(self, max_edges: int = 4096):
        self.max_edges = max_edges
        self.edges: Dict[Tuple[str, str], str] = {}

    def add_edge(self, src: str, dst: str, label: str = "") -> None:
        if (src, dst) not in self.edges and len(self.edges) >= self.max_edges:
            raise OverflowError("threat graph is full")
        self.edges[(src, dst)] = label

    def remove_edge(self, src: str, dst: str) -> bool:
        return self.edges.pop((src, dst), None) is not None

    def clear(self) -> None:
        self.edges.clear()

    def edge_count(self) -> int:
        return len(self.edges)

    def nodes(self) -> List[str]:
        return sorted({n for e in self.edges for n in e})

    def attack_paths(self, src: str, dst: str, max_len: int = 8) -> List[List[str]]:
        adj: Dict[str, List[str]] = {}
        for a, b in self.edges:
            adj.setdefault(a, []).append(b)
        out, stack = [], [(src, [src])]
        while stack:
            node, path = stack.pop()
            if node == dst:
                out.append(path)
                continue
            if len(path) > max_len:
                continue
            for nxt in sorted(adj.get(node, ()), reverse=True):
                if nxt not in path:
                    stack.append((nxt, path + [nxt]))
        return sorted(out, key=lambda p: (len(p), p))

    def choke_points(self, src: str, dst: str) -> List[str]:
        """Inner nodes that every attack path from ``src`` to ``dst`` passes through: hardening one of them cuts all."""
        paths = self.attack_paths(src, dst)
        if not paths:
            return []
        common = set(paths[0][1:-1])
        for p in paths[1:]:
            common &= set(p[1:-1])
        return sorted(common)

    def export_dot(self, path: Optional[str] = None) -> str:
        q = lambda s: '"' + s.replace("\\", "\\\\").replace('"', '\\"') + '"'          # noqa: E731
        lines = ["digraph threats {", "  rankdir=LR;"]
        lines += [f"  {q(a)} -> {q(b)}" + (f" [label={q(l)}]" if l else "") + ";" for (a, b), l in sorted(self.edges.items())]
        text = "\n".join(lines + ["}"]) + "\n"
        if path:
            with open(path, "w") as f:
                f.write(text)
        return text


# ------------------------------------------------------------------------------------------------ dashboard, reports
class SecurityDashboard:
    """Named widgets (``counter``, ``gauge``, ``table``, ``text``) that monitoring code updates and an operator page
    reads. ``update`` merges a JSON payload ``{"widget name": value, ...}``; ``status`` is the JSON snapshot;
    ``render_html`` a self-contained page (everything escaped)."""

    TYPES = ("counter", "gauge", "table", "text")

    def __init__(self, title: str = "Security", clock: Callable[[], float] = time.time):
        self.title, self.clock = title, clock
        self.widgets: Dict[str, dict] = {}
        self.updated = 0.0

    def add_widget(self, name: str, kind: str, data: Any = None) -> None:
        if kind not in self.TYPES:
            raise ValueError(f"unknown widget type {kind!r}")
        self.widgets[name] = {"type": kind, "data": data if data is not None else (0 if kind in ("counter", "gauge") else
                                                                                    [] if kind == "table" else "")}

    def remove_widget(self, name: str) -> bool:
        return self.widgets.pop(name, None) is not None

    def update(self, payload) -> int:
        """Applies ``{"name": value}``; a counter adds the value, other widgets are replaced. Returns how many widgets
        changed; unknown names are ignored."""
        data = json.loads(payload) if isinstance(payload, (str, bytes)) else dict(payload)
        n = 0
        for name, value in data.items():
            w = self.widgets.get(name)
            if w is None:
                continue
            w["data"] = w["data"] + value if w["type"] == "counter" else value
            n += 1
        if n:
            self.updated = self.clock()
        return n

    def status(self) -> str:
        return json.dumps({"title": self.title, "updated": self.updated, "widgets": self.widgets}, sort_keys=True, default=str)

    def render_html(self) -> str:
        rows = []
        for name, w in sorted(self.widgets.items()):
            if w["type"] == "table":
                body = "<table>" + "".join("<tr>" + "".join(f"<td>{html.escape(str(c))}</td>" for c in r) + "</tr>"
                                           for r in w["data"]) + "</table>"
            else:
                body = html.escape(str(w["data"]))
            rows.append(f'<section class="{w["type"]}"><h2>{html.escape(name)}</h2>{body}</section>')
        return f"<!doctype html><html><head><meta charset=\"utf-8\"><title>{html.escape(self.title)}</title></head><body>" \
               f"<h1>{html.escape(self.title)}</h1>{''.join(rows)}</body></html>"


class ComplianceReportBuilder:
    """Collects findings per control and writes the report as text, JSON or a one-page PDF. Statuses: ``pass``,
    ``fail``, ``partial``, ``n/a``; the score is passes plus half the partials over the applicable controls."""

    FRAMEWORKS = {"soc2": "SOC 2 Type II", "iso27001": "ISO/IEC 27001", "hipaa": "HIPAA Security Rule", "gdpr": "GDPR",
                  "pci-dss": "PCI DSS"}
    STATUSES = ("pass", "fail", "partial", "n/a")

    def __init__(self, company: str = ""):
        self.company = company
        self.findings: List[dict] = []

    def set_company(self, name: str) -> None:
        self.company = name

    def add_finding(self, control_id: str, status: str, description: str = "") -> None:
        if status not in self.STATUSES:
            raise ValueError(f"unknown status {status!r}")
        self.findings.append({"control": control_id, "status": status, "description": description})

    def score(self) -> float:
        live = [f for f in self.findings if f["status"] != "n/a"]
        if not live:
            return 1.0
        return sum({"pass": 1.0, "partial": 0.5}.get(f["status"], 0.0) for f in live) / len(live)

    def _lines(self, report_type: str) -> List[str]:
        if report_type not in self.FRAMEWORKS:
            raise ValueError(f"unknown report type {report_type!r}")
        head = [f"{self.FRAMEWORKS[report_type]} compliance report", f"Organisation: {self.company or '(not set)'}",
                f"Generated: {time.strftime('%Y-%m-%d %H:%M UTC', time.gmtime())}",
                f"Controls: {len(self.findings)}   Score: {self.score() * 100:.1f}%", ""]
        return head + [f"[{f['status'].upper():7s}] {f['control']}: {f['description']}" for f in self.findings]

    def generate(self, report_type: str, output_path: Optional[str] = None, fmt: str = "text") -> str:
        if fmt == "json":
            if report_type not in self.FRAMEWORKS:
                raise ValueError(f"unknown report type {report_type!r}")
            text = json.dumps({"framework": self.FRAMEWORKS[report_type], "company": self.company, "score": self.score(),
                               "findings": self.findings}, indent=2)
        else:
            text = "\n".join(self._lines(report_type)) + "\n"
        if output_path:
            with open(output_path, "w") as f:
                f.write(text)
        return text

    def generate_pdf(self, report_type: str, output_path: str) -> int:
        """A valid single-page PDF 1.4 (Helvetica, one text line per finding, long lines cut at 100 characters; lines
        beyond the page are dropped with a final "... n more"). Returns the file size."""
        lines = [l[:100] for l in self._lines(report_type)]
        if len(lines) > 52:
            lines = lines[:51] + [f"... {len(lines) - 51} more"]
        esc = lambda s: s.encode("latin-1", "replace").replace(b"\\", b"\\\\").replace(b"(", b"\\(").replace(b")", b"\\)")  # noqa: E731
        stream = b"BT /F1 10 Tf 50 780 Td 14 TL\n" + b"".join(b"(" + esc(l) + b") Tj T*\n" for l in lines) + b"ET\n"
        objs = [b"<< /Type /Catalog /Pages 2 0 R >>", b"<< /Type /Pages /Kids [3 0 R] /Count 1 >>",
                b"<< /Type /Page /Parent 2 0 R /MediaBox [0 0 612 842] /Contents 4 0 R /Resources << /Font << /F1 5 0 R >> >> >>",
                b"<< /Length " + str(len(stream)).encode() + b" >>\nstream\n" + stream + b"endstream",
                b"<< /Type /Font /Subtype /Type1 /BaseFont /Helvetica >>"]
        out, offsets = bytearray(b"%PDF-1.4\n"), []
        for i, o in enumerate(objs, 1):
            offsets.append(len(out))
            out += str(i).encode() + b" 0 obj\n" + o + b"\nendobj\n"
        xref = len(out)
        out += b"xref\n0 " + str(len(objs) + 1).encode() + b"\n0000000000 65535 f \n"
        out += b"".join(f"{off:010d} 00000 n \n".encode() for off in offsets)
        out += b"trailer\n<< /Size " + str(len(objs) + 1).encode() + b" /Root 1 0 R >>\nstartxref\n" + str(xref).encode() + b"\n%%EOF\n"
        with open(output_path, "wb") as f:
            f.write(out)
        return len(out)
