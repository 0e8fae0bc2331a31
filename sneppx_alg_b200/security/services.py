"""Security services S3-S9, host-side (the reference's ``security/`` tree and its Python bindings): integrity
monitor, token-bucket rate limiter / DDoS mitigation and firewall rules (S4), key vault and hash-chained audit log
(S6), signed updates with SBOM (S7), a small LTL checker over finite traces (S8), network-input fuzzer and
self-audit (S9), API-key store and usage tracker for the gateway."""
from __future__ import annotations

import hashlib
import ipaddress
import json
import os
import random
import re
import secrets
import time
from typing import Callable, Dict, List, Optional

from . import crypto


# ---- S3 integrity
class IntegrityMonitor:
    def __init__(self):
        self.baseline: Dict[str, str] = {}

    @staticmethod
    def _digest(path):
        with open(path, "rb") as f:
            return crypto.sha256(f.read()).hex()

    def snapshot(self, paths: List[str]):
        self.baseline = {p: self._digest(p) for p in paths}

    def verify(self) -> List[str]:
        bad = []
        for p, d in self.baseline.items():
            if not os.path.exists(p) or self._digest(p) != d:
                bad.append(p)
        return bad


# ---- S4 network
class TokenBucket:
    def __init__(self, rate: float, burst: float, clock: Callable[[], float] = time.monotonic):
        self.rate, self.burst, self.clock = rate, burst, clock
        self.tokens, self.t = burst, clock()

    def allow(self, cost: float = 1.0) -> bool:
        now = self.clock()
        self.tokens = min(self.burst, self.tokens + (now - self.t) * self.rate)
        self.t = now
        if self.tokens >= cost:
            self.tokens -= cost
            return True
        return False


class DDoSMitigator:
    """Per-client token buckets with temporary bans after repeated violations."""

    def __init__(self, rate=10.0, burst=20.0, ban_after=5, ban_seconds=60.0, clock=time.monotonic):
        self.rate, self.burst, self.ban_after, self.ban_seconds, self.clock = rate, burst, ban_after, ban_seconds, clock
        self.buckets: Dict[str, TokenBucket] = {}
        self.violations: Dict[str, int] = {}
        self.banned: Dict[str, float] = {}

    def check(self, client: str) -> bool:
        now = self.clock()
        if client in self.banned:
            if now < self.banned[client]:
                return False
            del self.banned[client]
            self.violations[client] = 0
        b = self.buckets.setdefault(client, TokenBucket(self.rate, self.burst, self.clock))
        if b.allow():
            return True
        self.violations[client] = self.violations.get(client, 0) + 1
        if self.violations[client] >= self.ban_after:
            self.banned[client] = now + self.ban_seconds
        return False


class Firewall:
    """Ordered allow / deny rules on source network and port; first match wins, default deny."""

    def __init__(self, default="deny"):
        self.rules, self.default = [], default

    def add_rule(self, action: str, cidr: str = "0.0.0.0/0", port: Optional[int] = None):
        self.rules.append((action, ipaddress.ip_network(cidr), port))

    def decide(self, src_ip: str, port: int) -> str:
        ip = ipaddress.ip_address(src_ip)
        for action, net, p in self.rules:
            if ip in net and (p is None or p == port):
                return action
        return self.default


# ---- S6 vault / audit
class KeyVault:
    """Secrets sealed with ChaCha20-Poly1305 under a key derived from the passphrase (PBKDF2-SHA256)."""

    def __init__(self, path: str, passphrase: str, iterations: int = 20000):
        self.path = path
        if os.path.exists(path):
            blob = json.load(open(path))
            self.salt = bytes.fromhex(blob["salt"])
            self.items = blob["items"]
            self.iterations = blob["iterations"]
        else:
            self.salt, self.items, self.iterations = secrets.token_bytes(16), {}, iterations
        self.key = crypto.pbkdf2_sha256(passphrase.encode(), self.salt, self.iterations)

    def put(self, name: str, secret: bytes):
        nonce = secrets.token_bytes(12)
        self.items[name] = {"nonce": nonce.hex(), "sealed": crypto.aead_encrypt(self.key, nonce, secret, name.encode()).hex()}
        self._flush()

    def get(self, name: str) -> bytes:
        it = self.items[name]
        return crypto.aead_decrypt(self.key, bytes.fromhex(it["nonce"]), bytes.fromhex(it["sealed"]), name.encode())

    def _flush(self):
        with open(self.path, "w") as f:
            json.dump({"salt": self.salt.hex(), "iterations": self.iterations, "items": self.items}, f)


class AuditLogger:
    """Tamper-evident log: every record carries the hash of the previous one."""

    def __init__(self, path: str):
        self.path = path
        self.last = "0" * 64
        if os.path.exists(path):
            for line in open(path):
                self.last = json.loads(line)["hash"]

    def log(self, actor: str, action: str, **details):
        rec = {"ts": time.time(), "actor": actor, "action": action, "details": details, "prev": self.last}
        rec["hash"] = crypto.sha256(json.dumps(rec, sort_keys=True).encode()).hex()
        self.last = rec["hash"]
        with open(self.path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        return rec["hash"]

    def verify(self) -> bool:
        prev = "0" * 64
        for line in open(self.path):
            rec = json.loads(line)
            h = rec.pop("hash")
            if rec["prev"] != prev or crypto.sha256(json.dumps(rec, sort_keys=True).encode()).hex() != h:
                return False
            prev = h
        return True


# ---- S7 updates
def sign_update(path: str, key: bytes, version: str, scheme: str = "hmac-sha256") -> dict:
    """Manifest for an update file. ``hmac-sha256``: `key` is a shared secret. ``ed25519``: `key` is the 32-byte
    signing seed and the manifest is verified with the public key only. ``ml-dsa-65``: `key` is the ML-DSA private
    key (post-quantum signature, FIPS 204), verified with its public key. ``slh-dsa-128f``: the hash-based
    SLH-DSA private key (FIPS 205; 17 KB signatures, security resting on SHAKE-256 alone)."""
    data = open(path, "rb").read()
    manifest = {"file": os.path.basename(path), "version": version, "sha256": crypto.sha256(data).hex(), "size": len(data),
                "scheme": scheme}
    payload = json.dumps(manifest, sort_keys=True).encode()
    if scheme == "ed25519":
        manifest["signature"] = crypto.ed25519_sign(key, payload).hex()
    elif scheme == "ml-dsa-65":
        manifest["signature"] = crypto.mldsa_sign(key, payload, 65, context=b"sneppx-update").hex()
    elif scheme == "slh-dsa-128f":
        manifest["signature"] = crypto.slhdsa_sign(key, payload, "128f", context=b"sneppx-update").hex()
    elif scheme == "hmac-sha256":
        manifest["signature"] = crypto.hmac_sha256(key, payload).hex()
    else:
        raise ValueError(f"unknown signature scheme {scheme!r}")
    return manifest


def verify_update(path: str, manifest: dict, key: bytes, min_version: str = "0") -> bool:
    """`key`: the shared secret (hmac-sha256) or the signer's public key (ed25519: 32 bytes; ml-dsa-65: 1952 bytes)."""
    m = dict(manifest)
    sig = bytes.fromhex(m.pop("signature"))
    payload = json.dumps(m, sort_keys=True).encode()
    if m.get("scheme", "hmac-sha256") == "ed25519":
        if not crypto.ed25519_verify(key, payload, sig):
            return False
    elif m.get("scheme") == "ml-dsa-65":
        if not crypto.mldsa_verify(key, payload, sig, 65, context=b"sneppx-update"):
            return False
    elif m.get("scheme") == "slh-dsa-128f":
        if not crypto.slhdsa_verify(key, payload, sig, "128f", context=b"sneppx-update"):
            return False
    elif not crypto.ct_equal(sig, crypto.hmac_sha256(key, payload)):
        return False
    data = open(path, "rb").read()
    as_tuple = lambda v: tuple(int(x) for x in re.findall(r"\d+", v))  # noqa: E731
    return crypto.sha256(data).hex() == m["sha256"] and len(data) == m["size"] and as_tuple(m["version"]) >= as_tuple(min_version)


def sbom(packages: Dict[str, str], known_cves: Dict[str, List[str]] = None) -> dict:
    """Software bill of materials with a vulnerability flag per component."""
    known_cves = known_cves or {}
    comps = [{"name": n, "version": v, "cves": known_cves.get(f"{n}=={v}", [])} for n, v in sorted(packages.items())]
    return {"components": comps, "vulnerable": [c["name"] for c in comps if c["cves"]]}


# ---- S8 formal: LTL over finite traces
def ltl_check(formula, trace: List[dict], i: int = 0) -> bool:
    """formula: ('ap', name) | ('not', f) | ('and', f, g) | ('or', f, g) | ('next', f) | ('always', f) |
    ('eventually', f) | ('until', f, g); finite-trace semantics."""
    op = formula[0]
    if op == "ap":
        return bool(trace[i].get(formula[1], False)) if i < len(trace) else False
    if op == "not":
        return not ltl_check(formula[1], trace, i)
    if op == "and":
        return ltl_check(formula[1], trace, i) and ltl_check(formula[2], trace, i)
    if op == "or":
        return ltl_check(formula[1], trace, i) or ltl_check(formula[2], trace, i)
    if op == "next":
        return i + 1 < len(trace) and ltl_check(formula[1], trace, i + 1)
    if op == "always":
        return all(ltl_check(formula[1], trace, j) for j in range(i, len(trace)))
    if op == "eventually":
        return any(ltl_check(formula[1], trace, j) for j in range(i, len(trace)))
    if op == "until":
        for j in range(i, len(trace)):
            if ltl_check(formula[2], trace, j):
                return True
            if not ltl_check(formula[1], trace, j):
                return False
        return False
    raise ValueError(op)


# ---- S9 pentest
def fuzz(target: Callable[[bytes], None], seeds: List[bytes], iterations=200, seed=0) -> List[dict]:
    """Mutation fuzzer: bit flips, truncation, duplication, interesting values; returns the crashing inputs."""
    rng, crashes = random.Random(seed), []
    for _ in range(iterations):
        data = bytearray(rng.choice(seeds))
        for _ in range(rng.randint(1, 4)):
            m = rng.randint(0, 3)
            if m == 0 and data:
                data[rng.randrange(len(data))] ^= 1 << rng.randrange(8)
            elif m == 1 and data:
                del data[rng.randrange(len(data)):]
            elif m == 2:
                data += data[: rng.randint(0, len(data))]
            else:
                pos = rng.randint(0, len(data))
                data[pos:pos] = rng.choice([b"\x00", b"\xff" * 4, b"%s%n", b"A" * 64, b"\x7f\xff\xff\xff"])
        try:
            target(bytes(data))
        except Exception as e:  # noqa: BLE001
            crashes.append({"input": bytes(data), "error": type(e).__name__})
    return crashes


def self_audit(config: dict) -> List[str]:
    findings = []
    if not config.get("api_keys_required", False):
        findings.append("API keys are not required")
    if config.get("bind", "127.0.0.1") == "0.0.0.0" and not config.get("tls", False):
        findings.append("listening on all interfaces without TLS")
    if config.get("max_prompt_chars", 0) <= 0:
        findings.append("no prompt size limit")
    if not config.get("audit_log"):
        findings.append("audit logging disabled")
    return findings


# ---- gateway helpers
class ApiKeyStore:
    def __init__(self):
        self.keys: Dict[str, dict] = {}

    def create(self, owner: str, scopes=("generate",)) -> str:
        k = "sk-" + secrets.token_hex(20)
        self.keys[hashlib.sha256(k.encode()).hexdigest()] = {"owner": owner, "scopes": list(scopes), "created": time.time(), "revoked": False}
        return k

    def check(self, key: str, scope: str = "generate") -> bool:
        rec = self.keys.get(hashlib.sha256(key.encode()).hexdigest())
        return bool(rec) and not rec["revoked"] and scope in rec["scopes"]

    def revoke(self, key: str):
        rec = self.keys.get(hashlib.sha256(key.encode()).hexdigest())
        if rec:
            rec["revoked"] = True


class UsageTracker:
    def __init__(self):
        self.usage: Dict[str, dict] = {}

    def record(self, owner: str, prompt_tokens: int, completion_tokens: int):
        u = self.usage.setdefault(owner, {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0})
        u["requests"] += 1
        u["prompt_tokens"] += prompt_tokens
        u["completion_tokens"] += completion_tokens

    def report(self, owner: str) -> dict:
        return dict(self.usage.get(owner, {}))


class ABSlots:
    """A/B slots for atomic updates of a deployed directory (``container_security.py:451-489`` keeps the slot of the
    boot partition; here the unit is a model / runtime directory): the inactive slot is filled and verified, then one
    atomic rename of the ``current`` marker makes it live, and ``rollback`` renames it back."""

    def __init__(self, root: str):
        self.root = root
        for s in ("_a", "_b"):
            os.makedirs(os.path.join(root, "slot" + s), exist_ok=True)
        if not os.path.exists(self._marker):
            self._write_marker("_a")

    @property
    def _marker(self) -> str:
        return os.path.join(self.root, "current")

    def _write_marker(self, slot: str):
        tmp = self._marker + ".tmp"
        with open(tmp, "w") as f:
            f.write(slot)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, self._marker)

    @property
    def current(self) -> str:
        return open(self._marker).read().strip()

    @property
    def inactive_slot(self) -> str:
        return "_b" if self.current == "_a" else "_a"

    def get_partition_path(self, partition: str = "", slot: Optional[str] = None) -> str:
        return os.path.join(self.root, "slot" + (slot or self.current), partition)

    def stage(self, name: str, data: bytes) -> str:
        """Writes a file into the inactive slot."""
        path = self.get_partition_path(name, self.inactive_slot)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "wb") as f:
            f.write(data)
        return path

    def switch_slot(self, verify: Optional[Callable[[str], bool]] = None) -> bool:
        """Makes the inactive slot live if `verify(slot directory)` accepts it (always, when no verifier is given)."""
        target = self.inactive_slot
        if verify is not None and not verify(self.get_partition_path("", target)):
            return False
        self._write_marker(target)
        return True

    rollback = switch_slot
