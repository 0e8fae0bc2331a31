"""Smaller security services: host-side chaos experiments, zero-trust access decisions, a hash-chained audit ledger
with quorum approval, threat-intelligence indicators, incident response with playbooks, compliance control checks,
measured-boot attestation and build provenance.

The reference declares these as interface headers without bodies (``security/chaos/fault_injection.h``,
``zero_trust/ztna_framework.h``, ``blockchain/consensus_audit.h``, ``threat_intel/*.h``, ``incident_response/*.h``,
``automation/soar_engine.h``, ``compliance/*_framework.h``, ``hardware/tee_interface.h``, ``supply_chain/sbom_manager.h``).
Everything here runs on the host; the chaos faults act on Python callables (exceptions, delays, dropped calls) and never
on a GPU.
"""
from __future__ import annotations

import json
import random
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

from . import crypto


# ------------------------------------------------------------------------------------------------- chaos
@dataclass
class Fault:
    """kind: "exception" (raise `error`), "delay" (sleep `delay_s`), "drop" (return `dropped` without calling).
    `probability` of firing per call, from a seeded generator so that runs repeat."""
    kind: str
    probability: float = 1.0
    delay_s: float = 0.0
    error: Exception = None
    dropped: object = None


class ChaosExperiment:
    """Steady-state hypothesis -> inject faults into named call sites -> probe -> roll back.

    ``wrap(name, fn)`` returns a callable that consults the experiment on every call; faults apply only while the
    experiment is running. ``run(workload)`` checks the probes before, runs the workload under faults, rolls back,
    checks the probes again and reports whether the hypothesis (all probes true) held."""

    def __init__(self, name: str, hypothesis: str = "", seed: int = 0):
        self.name, self.hypothesis = name, hypothesis
        self.faults: Dict[str, List[Fault]] = {}
        self.probes: Dict[str, Callable[[], bool]] = {}
        self.running = False
        self.rng = random.Random(seed)
        self.injected: Dict[str, int] = {}
        self.sleep = time.sleep

    def add_fault(self, site: str, fault: Fault):
        if fault.kind not in ("exception", "delay", "drop"):
            raise ValueError(f"unknown fault kind {fault.kind!r}")
        self.faults.setdefault(site, []).append(fault)

    def add_probe(self, name: str, fn: Callable[[], bool]):
        self.probes[name] = fn

    def wrap(self, site: str, fn: Callable) -> Callable:
        def wrapped(*a, **k):
            if self.running:
                for f in self.faults.get(site, ()):
                    if self.rng.random() < f.probability:
                        self.injected[site] = self.injected.get(site, 0) + 1
                        if f.kind == "exception":
                            raise f.error if f.error is not None else RuntimeError(f"chaos: injected failure at {site}")
                        if f.kind == "drop":
                            return f.dropped
                        self.sleep(f.delay_s)
            return fn(*a, **k)
        return wrapped

    def _probe_all(self) -> Dict[str, bool]:
        out = {}
        for n, fn in self.probes.items():
            try:
                out[n] = bool(fn())
            except Exception:
                out[n] = False
        return out

    def rollback(self):
        self.running = False

    def run(self, workload: Callable[[], object]) -> dict:
        before = self._probe_all()
        self.running, error = True, None
        try:
            workload()
        except Exception as e:                              # the workload failing under faults is a finding, not a crash
            error = repr(e)
        finally:
            self.rollback()
        after = self._probe_all()
        return {"experiment": self.name, "hypothesis": self.hypothesis, "steady_before": all(before.values()),
                "steady_after": all(after.values()), "hypothesis_valid": all(before.values()) and all(after.values()) and error is None,
                "workload_error": error, "injected": dict(self.injected), "probes": after}


# ------------------------------------------------------------------------------------------------- zero trust
@dataclass
class ZTPolicy:
    """Allow `actions` on resources matching `resource_prefix` to subjects holding all `roles`, at `min_trust` or
    above; rules are checked in order and the first match decides; no match means deny."""
    resource_prefix: str
    actions: Sequence[str]
    roles: Sequence[str] = ()
    min_trust: float = 0.0
    decision: str = "allow"


class ZeroTrustEngine:
    """Every request is decided from identity, device posture and context; nothing is trusted for being inside a
    network. A granted decision is a short-lived HMAC-signed token bound to (subject, resource, action)."""

    def __init__(self, key: bytes, token_ttl_s: float = 300.0):
        self.key, self.ttl = key, token_ttl_s
        self.policies: List[ZTPolicy] = []
        self.log: List[dict] = []

    def add_policy(self, p: ZTPolicy):
        self.policies.append(p)

    @staticmethod
    def trust_score(device: dict, context: dict) -> float:
        """0..1 from posture (disk encryption, patch level, managed) and context (MFA, known location, failures)."""
        s = 0.2
        s += 0.2 * bool(device.get("disk_encrypted")) + 0.15 * bool(device.get("managed")) + 0.15 * bool(device.get("patched"))
        s += 0.2 * bool(context.get("mfa")) + 0.1 * bool(context.get("known_location"))
        s -= 0.1 * min(int(context.get("recent_failures", 0)), 5)
        return max(0.0, min(1.0, s))

    def decide(self, subject: dict, resource: str, action: str, device: dict = None, context: dict = None, now: float = None) -> dict:
        now = time.time() if now is None else now
        trust = self.trust_score(device or {}, context or {})
        decision, why = "deny", "no matching policy"
        for p in self.policies:
            if resource.startswith(p.resource_prefix) and action in p.actions and set(p.roles) <= set(subject.get("roles", ())):
                if trust >= p.min_trust:
                    decision, why = p.decision, f"policy {p.resource_prefix}"
                else:
                    decision, why = "deny", f"trust {trust:.2f} below {p.min_trust:.2f}"
                break
        out = {"decision": decision, "reason": why, "trust": trust}
        if decision == "allow":
            body = json.dumps({"sub": subject.get("id"), "res": resource, "act": action, "exp": now + self.ttl}, sort_keys=True)
            out["token"] = body + "." + crypto.hmac_sha256(self.key, body.encode()).hex()
        self.log.append({"t": now, "sub": subject.get("id"), "res": resource, "act": action, **{k: out[k] for k in ("decision", "reason")}})
        return out

    def check_token(self, token: str, resource: str, action: str, now: float = None) -> bool:
        now = time.time() if now is None else now
        body, _, mac = token.rpartition(".")
        try:
            if not crypto.ct_equal(bytes.fromhex(mac), crypto.hmac_sha256(self.key, body.encode())):
                return False
            claims = json.loads(body)
        except ValueError:
            return False
        return claims.get("res") == resource and claims.get("act") == action and claims.get("exp", 0) > now


# ------------------------------------------------------------------------------------------------- audit ledger
def merkle_root(leaves: Sequence[bytes]) -> bytes:
    """SHA-256 Merkle root with domain-separated leaves (0x00) and nodes (0x01); an odd node is carried up."""
    level = [crypto.sha256(b"\x00" + x) for x in leaves] or [crypto.sha256(b"")]
    while len(level) > 1:
        nxt = [crypto.sha256(b"\x01" + level[i] + level[i + 1]) for i in range(0, len(level) - 1, 2)]
        if len(level) % 2:
            nxt.append(level[-1])
        level = nxt
    return level[0]


class AuditLedger:
    """Append-only ledger: each block commits to its records (Merkle root) and to the previous block's hash, and is
    final once a quorum of the registered validators has signed it (Ed25519). Any later change of a record, a block
    or their order breaks ``verify``."""

    def __init__(self, validators: Dict[str, bytes], quorum: Optional[int] = None):
        self.validators = dict(validators)                       # name -> Ed25519 public key
        self.quorum = quorum if quorum is not None else len(validators) * 2 // 3 + 1
        self.blocks: List[dict] = []
        self.pending: List[dict] = []

    def append(self, record: dict):
        self.pending.append(record)

    def propose(self, now: float = None) -> dict:
        leaves = [json.dumps(r, sort_keys=True).encode() for r in self.pending]
        prev = self.blocks[-1]["hash"] if self.blocks else "00" * 32
        head = {"index": len(self.blocks), "prev": prev, "root": merkle_root(leaves).hex(), "time": time.time() if now is None else now,
                "count": len(leaves)}
        block = {**head, "hash": crypto.sha256(json.dumps(head, sort_keys=True).encode()).hex(), "records": list(self.pending), "votes": {}}
        return block

    @staticmethod
    def vote(block: dict, name: str, seed: bytes):
        block["votes"][name] = crypto.ed25519_sign(seed, bytes.fromhex(block["hash"])).hex()

    def _valid_votes(self, block: dict) -> int:
        return sum(1 for n, s in block["votes"].items()
                   if n in self.validators and crypto.ed25519_verify(self.validators[n], bytes.fromhex(block["hash"]), bytes.fromhex(s)))

    def commit(self, block: dict) -> bool:
        if block["index"] != len(self.blocks) or self._valid_votes(block) < self.quorum:
            return False
        self.blocks.append(block)
        self.pending = []
        return True

    def verify(self) -> bool:
        prev = "00" * 32
        for i, b in enumerate(self.blocks):
            head = {k: b[k] for k in ("index", "prev", "root", "time", "count")}
            leaves = [json.dumps(r, sort_keys=True).encode() for r in b["records"]]
            if (b["index"] != i or b["prev"] != prev or b["root"] != merkle_root(leaves).hex() or b["count"] != len(leaves)
                    or b["hash"] != crypto.sha256(json.dumps(head, sort_keys=True).encode()).hex() or self._valid_votes(b) < self.quorum):
                return False
            prev = b["hash"]
        return True


# ------------------------------------------------------------------------------------------------- threat intelligence
class ThreatIntel:
    """Indicators of compromise (ip, domain, sha256, ...) with confidence, source and expiry; ``match`` enriches an
    event with the indicators it touches and a combined score 1 - prod(1 - confidence)."""

    def __init__(self):
        self.indicators: Dict[tuple, dict] = {}

    def add(self, kind: str, value: str, confidence: float = 0.5, source: str = "", ttl_s: float = 30 * 86400, now: float = None):
        now = time.time() if now is None else now
        key = (kind, value.lower())
        old = self.indicators.get(key)
        conf = max(confidence, old["confidence"]) if old else confidence
        self.indicators[key] = {"kind": kind, "value": value.lower(), "confidence": conf, "expires": now + ttl_s,
                                "sources": sorted(set((old["sources"] if old else []) + [source]))}

    def expire(self, now: float = None) -> int:
        now = time.time() if now is None else now
        dead = [k for k, v in self.indicators.items() if v["expires"] <= now]
        for k in dead:
            del self.indicators[k]
        return len(dead)

    def match(self, event: dict, now: float = None) -> dict:
        now = time.time() if now is None else now
        hits = [v for (kind, value), v in self.indicators.items() if v["expires"] > now and str(event.get(kind, "")).lower() == value]
        miss = 1.0
        for h in hits:
            miss *= 1.0 - h["confidence"]
        return {"hits": hits, "score": 1.0 - miss}


# ------------------------------------------------------------------------------------------------- incidents / SOAR
_STATES = ("open", "triaged", "contained", "resolved")


class IncidentManager:
    """Incident records with an ordered life cycle, evidence with digests, and playbooks: lists of (name, action)
    steps registered per incident type and run in order until one fails."""

    def __init__(self):
        self.incidents: Dict[int, dict] = {}
        self.playbooks: Dict[str, List[tuple]] = {}
        self._next = 1

    def register_playbook(self, incident_type: str, steps: Sequence[tuple]):
        self.playbooks[incident_type] = list(steps)

    def open(self, incident_type: str, severity: str, summary: str, now: float = None) -> int:
        if severity not in ("low", "medium", "high", "critical"):
            raise ValueError("severity must be low, medium, high or critical")
        i = self._next
        self._next += 1
        self.incidents[i] = {"id": i, "type": incident_type, "severity": severity, "summary": summary, "state": "open",
                             "opened": time.time() if now is None else now, "evidence": [], "timeline": [("open", summary)]}
        return i

    def advance(self, incident: int, state: str, note: str = ""):
        rec = self.incidents[incident]
        if _STATES.index(state) != _STATES.index(rec["state"]) + 1:
            raise ValueError(f"cannot go from {rec['state']} to {state}")
        rec["state"] = state
        rec["timeline"].append((state, note))

    def add_evidence(self, incident: int, name: str, data: bytes):
        self.incidents[incident]["evidence"].append({"name": name, "sha256": crypto.sha256(data).hex(), "size": len(data)})

    def run_playbook(self, incident: int) -> List[dict]:
        rec = self.incidents[incident]
        results = []
        for name, action in self.playbooks.get(rec["type"], ()):
            try:
                results.append({"step": name, "ok": True, "result": action(rec)})
            except Exception as e:
                results.append({"step": name, "ok": False, "error": repr(e)})
                break
        rec["timeline"].append(("playbook", [r["step"] + (":ok" if r["ok"] else ":failed") for r in results]))
        return results


# ------------------------------------------------------------------------------------------------- compliance
_CONTROLS = {
    "encryption_at_rest": lambda c: bool(c.get("encrypt_checkpoints") or c.get("encryption_at_rest")),
    "encryption_in_transit": lambda c: bool(c.get("tls") or c.get("secure_transport")),
    "access_control": lambda c: bool(c.get("api_keys_required") or c.get("auth_mode") == "api_key"),
    "audit_logging": lambda c: bool(c.get("audit_log")),
    "key_rotation": lambda c: 0 < float(c.get("key_rotation_days", 0)) <= 365,
    "data_retention": lambda c: float(c.get("retention_days", 0)) > 0,
    "erasure": lambda c: bool(c.get("supports_erasure")),
    "mfa": lambda c: bool(c.get("mfa")),
    "vulnerability_management": lambda c: bool(c.get("sbom") or c.get("cve_scan")),
    "incident_response": lambda c: bool(c.get("incident_contact")),
}
FRAMEWORKS = {
    "gdpr": ("encryption_at_rest", "encryption_in_transit", "access_control", "audit_logging", "data_retention", "erasure"),
    "hipaa": ("encryption_at_rest", "encryption_in_transit", "access_control", "audit_logging", "incident_response"),
    "soc2": ("access_control", "audit_logging", "key_rotation", "vulnerability_management", "incident_response", "encryption_in_transit"),
    "pci_dss": ("encryption_at_rest", "encryption_in_transit", "access_control", "audit_logging", "key_rotation", "mfa",
                "vulnerability_management"),
    "fedramp": tuple(_CONTROLS),
}


def compliance_report(config: dict, framework: str) -> dict:
    """Which controls of `framework` (gdpr, hipaa, soc2, pci_dss, fedramp) the deployment configuration satisfies."""
    if framework not in FRAMEWORKS:
        raise ValueError(f"unknown framework {framework!r}; known: {sorted(FRAMEWORKS)}")
    results = {c: bool(_CONTROLS[c](config)) for c in FRAMEWORKS[framework]}
    return {"framework": framework, "controls": results, "passed": sum(results.values()), "total": len(results),
            "compliant": all(results.values()), "missing": [c for c, ok in results.items() if not ok]}


# ------------------------------------------------------------------------------------------------- attestation / provenance
class MeasuredBoot:
    """Platform-configuration-register style measurement: ``extend`` folds each component digest into a running hash
    in order; a quote signs (value, nonce) with the device key so that a verifier holding the expected component list
    can tell whether exactly those components were loaded in that order."""

    def __init__(self):
        self.value = bytes(32)
        self.log: List[tuple] = []

    def extend(self, name: str, data: bytes):
        d = crypto.sha256(data)
        self.value = crypto.sha256(self.value + d)
        self.log.append((name, d.hex()))

    def quote(self, device_seed: bytes, nonce: bytes) -> dict:
        return {"value": self.value.hex(), "nonce": nonce.hex(), "signature": crypto.ed25519_sign(device_seed, self.value + nonce).hex()}

    @staticmethod
    def expected(components: Sequence[bytes]) -> bytes:
        v = bytes(32)
        for c in components:
            v = crypto.sha256(v + crypto.sha256(c))
        return v

    @staticmethod
    def verify_quote(quote: dict, device_public: bytes, nonce: bytes, components: Sequence[bytes]) -> bool:
        value = bytes.fromhex(quote["value"])
        return (quote["nonce"] == nonce.hex() and value == MeasuredBoot.expected(components)
                and crypto.ed25519_verify(device_public, value + nonce, bytes.fromhex(quote["signature"])))


def provenance_attestation(artifacts: Dict[str, bytes], builder: str, source: str, seed: bytes) -> dict:
    """Signed statement of which artifacts (by SHA-256) a builder produced from which source revision."""
    body = {"builder": builder, "source": source, "subjects": {n: crypto.sha256(d).hex() for n, d in sorted(artifacts.items())}}
    return {**body, "signature": crypto.ed25519_sign(seed, json.dumps(body, sort_keys=True).encode()).hex()}


def verify_provenance(att: dict, artifacts: Dict[str, bytes], public: bytes) -> bool:
    body = {k: att[k] for k in ("builder", "source", "subjects")}
    if not crypto.ed25519_verify(public, json.dumps(body, sort_keys=True).encode(), bytes.fromhex(att["signature"])):
        return False
    return all(att["subjects"].get(n) == crypto.sha256(d).hex() for n, d in artifacts.items()) and set(artifacts) == set(att["subjects"])
