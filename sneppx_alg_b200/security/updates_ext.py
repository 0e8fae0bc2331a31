"""S7 extensions: what it takes to ship an update to a fleet and trust it on arrival.

* ``TufRepository`` / ``TufClient``: the four-role metadata scheme of The Update Framework (root, targets, snapshot,
  timestamp) on Ed25519 with thresholds, versions, expiry, root rotation and rollback / freeze / mix-and-match checks;
* ``bsdiff`` / ``bspatch``: binary deltas in the BSDIFF40 container (bzip2-compressed control, diff and extra blocks);
  ``bsdiff_signed`` adds a detached Ed25519 signature;
* ``Manifest``: file list with sizes and SHA-256, signed, verified file by file;
* ``SoftTpm``: PCR bank with extend / read, signed quotes over a nonce, sealing bound to a PCR selection, variables;
* ``ABPartition``: A/B slots with good / bad marks, boot attempt counting and automatic fallback;
* ``CanaryRollout``: staged percentages with a deterministic cohort per unit and a health gate on promotion;
* ``OfflineBundle``: one signed file carrying payloads and their manifest for air-gapped installs;
* ``DepResolver``: version selection under semver-style constraints by backtracking, with an install order.

Reference behaviour: security/updates/s7_extensions.c (function families ``tuf_*``, ``bsdiff*`` / ``bspatch*``,
``manifest_*``, ``tpm_*``, ``ab_*``, ``canary_rollout_*``, ``offline_bundle_*``, ``dep_resolver_*``). Signed update
manifests with HMAC / Ed25519 / ML-DSA / SLH-DSA signatures and the SBOM are in ``security/services.py``.
"""
from __future__ import annotations

import bz2
import hashlib
import json
import os
import struct
import time
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from . import crypto


def canonical_json(obj: Any) -> bytes:
    """Deterministic encoding that signatures are computed over: sorted keys, no insignificant white space."""
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=True).encode()


# ------------------------------------------------------------------------------------------------ TUF
TUF_ROLES = ("root", "targets", "snapshot", "timestamp")


class TufError(RuntimeError):
    pass


def _keyid(public: bytes) -> str:
    return hashlib.sha256(public).hexdigest()


def _sign_metadata(signed: dict, seeds: Iterable[bytes]) -> dict:
    body = canonical_json(signed)
    return {"signed": signed, "signatures": [{"keyid": _keyid(crypto.ed25519_public_key(s)),
                                              "sig": crypto.ed25519_sign(s, body).hex()} for s in seeds]}


def _verify_metadata(meta: dict, role: str, root_signed: dict) -> None:
    """Raises unless ``meta`` carries at least the role's threshold of valid signatures by distinct keys that the
    given root lists for that role."""
    spec = root_signed["roles"][role]
    body = canonical_json(meta["signed"])
    good = set()
    for s in meta.get("signatures", ()):
        kid = s.get("keyid")
        if kid in spec["keyids"] and kid in root_signed["keys"] and kid not in good:
            try:
                if crypto.ed25519_verify(bytes.fromhex(root_signed["keys"][kid]), body, bytes.fromhex(s["sig"])):
                    good.add(kid)
            except ValueError:
                pass
    if len(good) < spec["threshold"]:
        raise TufError(f"{role}: {len(good)} valid signatures, threshold {spec['threshold']}")
    if meta["signed"].get("_type") != role:
        raise TufError(f"{role}: metadata is of type {meta['signed'].get('_type')!r}")


class TufRepository:
    """The publishing side. Holds the role keys (Ed25519 seeds), the target files and produces signed metadata.
    ``publish`` bumps targets / snapshot / timestamp; ``rotate_key`` issues a new root signed by the old and the new
    root keys."""

    def __init__(self, thresholds: Optional[Dict[str, int]] = None, keys_per_role: Optional[Dict[str, int]] = None,
                 clock: Callable[[], float] = time.time, lifetime_s: Optional[Dict[str, float]] = None):
        self.clock = clock
        self.thresholds = {r: 1 for r in TUF_ROLES} | (thresholds or {})
        n = {r: self.thresholds[r] for r in TUF_ROLES} | (keys_per_role or {})
        self.seeds: Dict[str, List[bytes]] = {r: [os.urandom(32) for _ in range(n[r])] for r in TUF_ROLES}
        self.lifetime_s = {"root": 365 * 86400.0, "targets": 90 * 86400.0, "snapshot": 7 * 86400.0, "timestamp": 86400.0} | (lifetime_s or {})
        self.targets: Dict[str, bytes] = {}
        self.versions = {r: 0 for r in TUF_ROLES}
        self.metadata: Dict[str, dict] = {}
        self.root_history: List[dict] = []
        self._new_root(self.seeds["root"])
        self.publish()

    def _expires(self, role: str) -> float:
        return self.clock() + self.lifetime_s[role]

    def _new_root(self, signers: Sequence[bytes]) -> None:
        self.versions["root"] += 1
        keys, roles = {}, {}
        for r in TUF_ROLES:
            pubs = [crypto.ed25519_public_key(s) for s in self.seeds[r]]
            keys.update({_keyid(p): p.hex() for p in pubs})
            roles[r] = {"keyids": [_keyid(p) for p in pubs], "threshold": self.thresholds[r]}
        signed = {"_type": "root", "version": self.versions["root"], "expires": self._expires("root"), "keys": keys, "roles": roles}
        self.metadata["root"] = _sign_metadata(signed, signers)
        self.root_history.append(self.metadata["root"])

    def add_target(self, name: str, data: bytes) -> None:
        self.targets[name] = bytes(data)

    def remove_target(self, name: str) -> bool:
        return self.targets.pop(name, None) is not None

    @staticmethod
    def _describe(raw: bytes) -> dict:
        return {"length": len(raw), "hashes": {"sha256": hashlib.sha256(raw).hexdigest()}}

    def publish(self) -> None:
        for r in ("targets", "snapshot", "timestamp"):
            self.versions[r] += 1
        t = {"_type": "targets", "version": self.versions["targets"], "expires": self._expires("targets"),
             "targets": {n: self._describe(d) for n, d in sorted(self.targets.items())}}
        self.metadata["targets"] = _sign_metadata(t, self.seeds["targets"])
        s = {"_type": "snapshot", "version": self.versions["snapshot"], "expires": self._expires("snapshot"),
             "meta": {"targets.json": {"version": t["version"], **self._describe(canonical_json(self.metadata["targets"]))}}}
        self.metadata["snapshot"] = _sign_metadata(s, self.seeds["snapshot"])
        self.refresh_timestamp(bump=False)

    def refresh_timestamp(self, bump: bool = True) -> None:
        if bump:
            self.versions["timestamp"] += 1
        ts = {"_type": "timestamp", "version": self.versions["timestamp"], "expires": self._expires("timestamp"),
              "meta": {"snapshot.json": {"version": self.versions["snapshot"],
                                         **self._describe(canonical_json(self.metadata["snapshot"]))}}}
        self.metadata["timestamp"] = _sign_metadata(ts, self.seeds["timestamp"])

    def rotate_key(self, role: str, index: int = 0) -> None:
        """Replaces one key of ``role`` (revoking the old one). The new root is signed by the previous root keys and,
        when the root role itself changed, also by the new ones, so that a client can walk from either."""
        old_root = list(self.seeds["root"])
        self.seeds[role][index] = os.urandom(32)
        signers = {s: None for s in old_root + self.seeds["root"]}
        self._new_root(list(signers))
        self.publish()

    def fetch(self, role: str, root_version: Optional[int] = None) -> dict:
        if role == "root" and root_version is not None:
            if not 1 <= root_version <= len(self.root_history):
                raise KeyError(root_version)
            return self.root_history[root_version - 1]
        return self.metadata[role]

    def fetch_target(self, name: str) -> bytes:
        return self.targets[name]


class TufClient:
    """The consuming side, started from a trusted root. ``refresh`` runs the update workflow of the TUF specification
    (section 5.3 onward): walk the root chain, then timestamp, snapshot and targets, each checked for signatures,
    expiry, version regressions and agreement with the metadata above it. ``download`` checks a target's length and
    hash against the trusted targets metadata."""

    MAX_ROOT_ROTATIONS = 64

    def __init__(self, trusted_root: dict, clock: Callable[[], float] = time.time):
        _verify_metadata(trusted_root, "root", trusted_root["signed"])
        self.clock = clock
        self.trusted: Dict[str, dict] = {"root": trusted_root}

    def _fresh(self, meta: dict, role: str) -> None:
        if meta["signed"]["expires"] <= self.clock():
            raise TufError(f"{role}: metadata has expired")

    def _no_rollback(self, meta: dict, role: str) -> None:
        old = self.trusted.get(role)
        if old is not None and meta["signed"]["version"] < old["signed"]["version"]:
            raise TufError(f"{role}: version went back from {old['signed']['version']} to {meta['signed']['version']}")

    @staticmethod
    def _matches(meta: dict, described: dict, role: str) -> None:
        raw = canonical_json(meta)
        if described.get("version") != meta["signed"]["version"]:
            raise TufError(f"{role}: version {meta['signed']['version']} is not the one listed ({described.get('version')})")
        if "hashes" in described and (len(raw) != described["length"] or
                                      hashlib.sha256(raw).hexdigest() != described["hashes"]["sha256"]):
            raise TufError(f"{role}: content does not match the hash listed for it")

    def refresh(self, repo) -> Dict[str, int]:
        root = self.trusted["root"]
        for _ in range(self.MAX_ROOT_ROTATIONS):
            try:
                nxt = repo.fetch("root", root["signed"]["version"] + 1)
            except KeyError:
                break
            _verify_metadata(nxt, "root", root["signed"])          # trusted by the root we hold ...
            _verify_metadata(nxt, "root", nxt["signed"])           # ... and consistent with itself
            if nxt["signed"]["version"] != root["signed"]["version"] + 1:
                raise TufError("root: versions must increase by one")
            for r in ("timestamp", "snapshot"):                    # a rotated key invalidates what it signed (fast-forward recovery)
                if root["signed"]["roles"][r]["keyids"] != nxt["signed"]["roles"][r]["keyids"]:
                    self.trusted.pop("timestamp", None)
                    self.trusted.pop("snapshot", None)
            root = nxt
        self._fresh(root, "root")
        self.trusted["root"] = root
        rs = root["signed"]
        ts = repo.fetch("timestamp")
        _verify_metadata(ts, "timestamp", rs)
        self._no_rollback(ts, "timestamp")
        self._fresh(ts, "timestamp")
        snap = repo.fetch("snapshot")
        _verify_metadata(snap, "snapshot", rs)
        self._matches(snap, ts["signed"]["meta"]["snapshot.json"], "snapshot")
        self._no_rollback(snap, "snapshot")
        old_snap = self.trusted.get("snapshot")
        if old_snap is not None:
            for name, d in old_snap["signed"]["meta"].items():
                new = snap["signed"]["meta"].get(name)
                if new is None or new["version"] < d["version"]:
                    raise TufError(f"snapshot: {name} went back or disappeared")
        self._fresh(snap, "snapshot")
        tg = repo.fetch("targets")
        _verify_metadata(tg, "targets", rs)
        self._matches(tg, snap["signed"]["meta"]["targets.json"], "targets")
        self._no_rollback(tg, "targets")
        self._fresh(tg, "targets")
        self.trusted.update(timestamp=ts, snapshot=snap, targets=tg)
        return {r: self.trusted[r]["signed"]["version"] for r in TUF_ROLES}

    def target_info(self, name: str) -> Optional[dict]:
        tg = self.trusted.get("targets")
        return None if tg is None else tg["signed"]["targets"].get(name)

    def download(self, repo, name: str) -> bytes:
        info = self.target_info(name)
        if info is None:
            raise TufError(f"{name}: not a trusted target")
        raw = repo.fetch_target(name)
        if len(raw) != info["length"] or hashlib.sha256(raw).hexdigest() != info["hashes"]["sha256"]:
            raise TufError(f"{name}: length or hash does not match the targets metadata")
        return raw


# ------------------------------------------------------------------------------------------------ binary deltas
def _offtout(x: int) -> bytes:
    """bsdiff's 8-byte integer: little-endian magnitude with the sign in the top bit."""
    return struct.pack("<Q", (-x) | (1 << 63) if x < 0 else x)


def _offtin(b: bytes) -> int:
    v = struct.unpack("<Q", b)[0]
    return -(v & ((1 << 63) - 1)) if v >> 63 else v


def bsdiff(old: bytes, new: bytes, anchor: int = 12) -> bytes:
    """A BSDIFF40 patch taking ``old`` to ``new``. Matching regions are found from exact ``anchor``-byte seeds (hash
    index over ``old``) and grown in both directions through scattered differences, which end up as small numbers in
    the diff block (new minus old, byte-wise) and compress away; everything else goes to the extra block."""
    index: Dict[bytes, List[int]] = {}
    for i in range(0, max(0, len(old) - anchor + 1)):
        index.setdefault(old[i:i + anchor], []).append(i)
    ctrl, diff, extra = bytearray(), bytearray(), bytearray()
    old_pos = 0                         # where the patcher's old cursor stands
    pending_extra = bytearray()
    last_diff_len = 0
    records: List[List[int]] = []       # [diff_len, extra_len, seek] being assembled
    n = 0
    while n < len(new):
        cands = index.get(new[n:n + anchor]) if n + anchor <= len(new) else None
        if not cands:
            pending_extra.append(new[n])
            n += 1
            continue
        best_o, best_len = -1, 0
        for o in cands[:32]:
            # forward extension with a mismatch budget: stop when the recent window is mostly mismatches
            l, score, best_here, best_score = anchor, anchor, anchor, anchor
            while n + l < len(new) and o + l < len(old):
                score += 1 if new[n + l] == old[o + l] else -1
                l += 1
                if score > best_score:
                    best_score, best_here = score, l
                if score < best_score - 16:
                    break
            if best_here > best_len:
                best_o, best_len = o, best_here
        # backward extension into bytes that were about to become "extra"
        back = 0
        while back < len(pending_extra) and best_o - back - 1 >= 0 and \
                pending_extra[len(pending_extra) - 1 - back] == old[best_o - back - 1]:
            back += 1
        if back:
            del pending_extra[len(pending_extra) - back:]
            n, best_o, best_len = n - back, best_o - back, best_len + back
        if records:
            records[-1][1] = len(pending_extra)
            records[-1][2] = best_o - old_pos
        else:
            records.append([0, len(pending_extra), best_o])
        extra += pending_extra
        pending_extra = bytearray()
        records.append([best_len, 0, 0])
        diff += bytes((new[n + i] - old[best_o + i]) & 0xFF for i in range(best_len))
        old_pos = best_o + best_len
        n += best_len
    if not records:
        records.append([0, 0, 0])
    records[-1][1] = len(pending_extra)
    extra += pending_extra
    for d, e, s in records:
        ctrl += _offtout(d) + _offtout(e) + _offtout(s)
    cz, dz, ez = bz2.compress(bytes(ctrl)), bz2.compress(bytes(diff)), bz2.compress(bytes(extra))
    return b"BSDIFF40" + _offtout(len(cz)) + _offtout(len(dz)) + _offtout(len(new)) + cz + dz + ez


def bsdiff_total_size(patch: bytes) -> int:
    """Size of the file the patch produces (from the header)."""
    if len(patch) < 32 or patch[:8] != b"BSDIFF40":
        raise ValueError("not a BSDIFF40 patch")
    return _offtin(patch[24:32])


def bspatch(old: bytes, patch: bytes) -> bytes:
    """Applies a BSDIFF40 patch (from ``bsdiff`` here or from the original tool)."""
    new_size = bsdiff_total_size(patch)
    clen, dlen = _offtin(patch[8:16]), _offtin(patch[16:24])
    if clen < 0 or dlen < 0 or new_size < 0 or 32 + clen + dlen > len(patch):
        raise ValueError("corrupt patch header")
    ctrl = bz2.decompress(patch[32:32 + clen])
    diff = bz2.decompress(patch[32 + clen:32 + clen + dlen])
    extra = bz2.decompress(patch[32 + clen + dlen:])
    out = bytearray()
    op = dp = ep = 0
    for c in range(0, len(ctrl), 24):
        if c + 24 > len(ctrl):
            raise ValueError("corrupt patch: truncated control block")
        x, y, z = _offtin(ctrl[c:c + 8]), _offtin(ctrl[c + 8:c + 16]), _offtin(ctrl[c + 16:c + 24])
        if x < 0 or y < 0 or len(out) + x + y > new_size or dp + x > len(diff) or ep + y > len(extra):
            raise ValueError("corrupt patch: block sizes")
        for i in range(x):
            o = old[op + i] if 0 <= op + i < len(old) else 0
            out.append((diff[dp + i] + o) & 0xFF)
        op, dp = op + x, dp + x
        out += extra[ep:ep + y]
        ep += y
        op += z
    if len(out) != new_size:
        raise ValueError("corrupt patch: wrong output size")
    return bytes(out)


def bsdiff_signed(old: bytes, new: bytes, signing_seed: bytes) -> Tuple[bytes, bytes]:
    """(patch, Ed25519 signature over SHA-256(old) || SHA-256(new) || patch): the signature pins both ends."""
    patch = bsdiff(old, new)
    msg = hashlib.sha256(old).digest() + hashlib.sha256(new).digest() + patch
    return patch, crypto.ed25519_sign(signing_seed, msg)


def bspatch_verified(old: bytes, patch: bytes, signature: bytes, public_key: bytes) -> bytes:
    new = bspatch(old, patch)
    msg = hashlib.sha256(old).digest() + hashlib.sha256(new).digest() + patch
    if len(signature) != 64 or not crypto.ed25519_verify(public_key, msg, signature):
        raise ValueError("patch signature does not verify")
    return new


def bsdiff_files(old_path: str, new_path: str, patch_path: str) -> int:
    with open(old_path, "rb") as a, open(new_path, "rb") as b:
        patch = bsdiff(a.read(), b.read())
    with open(patch_path, "wb") as f:
        f.write(patch)
    return len(patch)


def bspatch_files(old_path: str, patch_path: str, new_path: str) -> int:
    with open(old_path, "rb") as a, open(patch_path, "rb") as p:
        new = bspatch(a.read(), p.read())
    tmp = new_path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(new)
    os.replace(tmp, new_path)
    return len(new)


# ------------------------------------------------------------------------------------------------ manifests
class Manifest:
    """File list of a release directory: relative path, size and SHA-256 per file, in sorted order, as canonical
    JSON. ``sign`` / ``verify`` use Ed25519 over the canonical bytes; ``verify_all`` also re-hashes every file."""

    def __init__(self, files: Optional[Dict[str, dict]] = None, meta: Optional[dict] = None):
        self.files, self.meta = dict(files or {}), dict(meta or {})

    @classmethod
    def create(cls, root: str, files: Optional[Iterable[str]] = None, meta: Optional[dict] = None) -> "Manifest":
        if files is None:
            files = [os.path.relpath(os.path.join(d, f), root) for d, _, fs in os.walk(root) for f in fs]
        out = {}
        for rel in sorted(files):
            if os.path.isabs(rel) or ".." in rel.replace("\\", "/").split("/"):
                raise ValueError(f"manifest paths stay inside the root: {rel!r}")
            h, size = hashlib.sha256(), 0
            with open(os.path.join(root, rel), "rb") as f:
                for chunk in iter(lambda: f.read(1 << 20), b""):
                    h.update(chunk)
                    size += len(chunk)
            out[rel.replace("\\", "/")] = {"size": size, "sha256": h.hexdigest()}
        return cls(out, meta)

    def encode(self) -> bytes:
        return canonical_json({"files": self.files, "meta": self.meta})

    @classmethod
    def decode(cls, raw: bytes) -> "Manifest":
        d = json.loads(raw)
        return cls(d["files"], d.get("meta"))

    def digest(self) -> bytes:
        return hashlib.sha256(self.encode()).digest()

    def sign(self, seed: bytes) -> bytes:
        return crypto.ed25519_sign(seed, self.encode())

    def verify(self, signature: bytes, public_key: bytes) -> bool:
        return len(signature) == 64 and crypto.ed25519_verify(public_key, self.encode(), signature)

    def check_files(self, root: str) -> List[str]:
        """Problems found under ``root``: missing files, wrong sizes, wrong hashes, files the manifest does not list."""
        problems = []
        for rel, want in self.files.items():
            path = os.path.join(root, rel)
            if not os.path.isfile(path):
                problems.append(f"missing: {rel}")
                continue
            got = Manifest.create(root, [rel]).files[rel]
            if got["size"] != want["size"]:
                problems.append(f"size: {rel}")
            elif got["sha256"] != want["sha256"]:
                problems.append(f"hash: {rel}")
        listed = set(self.files)
        for d, _, fs in os.walk(root):
            for f in fs:
                rel = os.path.relpath(os.path.join(d, f), root).replace("\\", "/")
                if rel not in listed:
                    problems.append(f"unlisted: {rel}")
        return sorted(problems)

    def verify_all(self, root: str, signature: bytes, public_key: bytes) -> bool:
        return self.verify(signature, public_key) and not self.check_files(root)


# ------------------------------------------------------------------------------------------------ software TPM
class TpmError(RuntimeError):
    pass


class SoftTpm:
    """The measured-boot subset of a TPM 2.0 in software: 24 SHA-256 PCRs (``extend`` folds a digest in, nothing sets
    one back short of ``reset``), quotes (the attestation key signs the nonce and a digest of the selected PCRs),
    sealing (data encrypted under a key derived from the storage root and the selected PCR values: it opens only
    while those PCRs hold the same values) and numbered variables."""

    NUM_PCRS = 24

    def __init__(self, endorsement_seed: Optional[bytes] = None):
        seed = endorsement_seed or os.urandom(32)
        self._srk = crypto.hkdf_sha256(seed, b"soft-tpm", b"storage root", 32)
        self._ak = crypto.hkdf_sha256(seed, b"soft-tpm", b"attestation", 32)
        self.pcrs = [b"\0" * 32 for _ in range(self.NUM_PCRS)]
        self.variables: Dict[int, int] = {}
        self.log: List[Tuple[int, bytes, str]] = []

    @property
    def attestation_public(self) -> bytes:
        return crypto.ed25519_public_key(self._ak)

    def _check(self, index: int) -> None:
        if not 0 <= index < self.NUM_PCRS:
            raise TpmError(f"PCR index {index} out of range")

    def pcr_read(self, index: int) -> bytes:
        self._check(index)
        return self.pcrs[index]

    def extend(self, index: int, digest: bytes, description: str = "") -> bytes:
        self._check(index)
        if len(digest) != 32:
            raise TpmError("a SHA-256 bank extends by 32-byte digests")
        self.pcrs[index] = hashlib.sha256(self.pcrs[index] + digest).digest()
        self.log.append((index, digest, description))
        return self.pcrs[index]

    def measure(self, index: int, data: bytes, description: str = "") -> bytes:
        return self.extend(index, hashlib.sha256(data).digest(), description)

    def reset(self) -> None:
        self.pcrs = [b"\0" * 32 for _ in range(self.NUM_PCRS)]
        self.log = []

    def _composite(self, mask: int) -> bytes:
        if mask <= 0 or mask >> self.NUM_PCRS:
            raise TpmError("PCR mask selects nothing or goes past the bank")
        h = hashlib.sha256(struct.pack(">I", mask))
        for i in range(self.NUM_PCRS):
            if mask >> i & 1:
                h.update(self.pcrs[i])
        return h.digest()

    def quote(self, nonce: bytes, pcr_mask: int) -> dict:
        comp = self._composite(pcr_mask)
        body = b"TPM-QUOTE" + struct.pack(">I", pcr_mask) + comp + hashlib.sha256(nonce).digest()
        return {"pcr_mask": pcr_mask, "composite": comp, "nonce": nonce, "signature": crypto.ed25519_sign(self._ak, body)}

    @staticmethod
    def verify_quote(quote: dict, attestation_public: bytes, nonce: bytes, expected_pcrs: Optional[Dict[int, bytes]] = None) -> bool:
        """Signature and nonce check; with ``expected_pcrs`` (index -> value for exactly the PCRs of the mask) also
        that the quoted composite is the one those values give."""
        if quote.get("nonce") != nonce:
            return False
        body = b"TPM-QUOTE" + struct.pack(">I", quote["pcr_mask"]) + quote["composite"] + hashlib.sha256(nonce).digest()
        if not crypto.ed25519_verify(attestation_public, body, quote["signature"]):
            return False
        if expected_pcrs is not None:
            mask = quote["pcr_mask"]
            if sorted(expected_pcrs) != [i for i in range(SoftTpm.NUM_PCRS) if mask >> i & 1]:
                return False
            h = hashlib.sha256(struct.pack(">I", mask))
            for i in sorted(expected_pcrs):
                h.update(expected_pcrs[i])
            return h.digest() == quote["composite"]
        return True

    @staticmethod
    def replay_log(log: Iterable[Tuple[int, bytes, str]]) -> Dict[int, bytes]:
        """PCR values that an event log leads to, for comparing with a quote."""
        pcrs: Dict[int, bytes] = {}
        for index, digest, _ in log:
            pcrs[index] = hashlib.sha256(pcrs.get(index, b"\0" * 32) + digest).digest()
        return pcrs

    def seal(self, data: bytes, pcr_mask: int) -> bytes:
        key = crypto.hkdf_sha256(self._srk, self._composite(pcr_mask), b"seal", 32)
        nonce = os.urandom(12)
        return struct.pack(">I", pcr_mask) + nonce + crypto.aead_encrypt(key, nonce, data, struct.pack(">I", pcr_mask))

    def unseal(self, sealed: bytes) -> bytes:
        if len(sealed) < 32:
            raise TpmError("sealed blob too short")
        mask = struct.unpack(">I", sealed[:4])[0]
        key = crypto.hkdf_sha256(self._srk, self._composite(mask), b"seal", 32)
        try:
            return crypto.aead_decrypt(key, sealed[4:16], sealed[16:], sealed[:4])
        except ValueError as e:
            raise TpmError("PCR state differs from the one the data was sealed to") from e

    def set_variable(self, index: int, value: int) -> None:
        self.variables[index] = value & 0xFFFFFFFF

    def get_variable(self, index: int) -> int:
        return self.variables.get(index, 0)


# ------------------------------------------------------------------------------------------------ A/B slots
class ABPartition:
    """Two system slots. An update is written to the inactive slot and ``swap`` makes it the boot target with
    ``max_tries`` boot attempts; the new system calls ``mark_good`` once it is up. ``boot`` is what the boot loader
    does on every start: count the attempt, and fall back to the other slot when the attempts are used up or the slot
    is marked bad."""

    def __init__(self, max_tries: int = 3):
        self.max_tries = max_tries
        self.active = 0
        self.good = [True, False]
        self.bad = [False, False]
        self.tries = [0, 0]
        self.versions = ["", ""]
        self.swap_ready = False

    @property
    def inactive(self) -> int:
        return 1 - self.active

    def write_inactive(self, version: str) -> int:
        s = self.inactive
        self.versions[s], self.good[s], self.bad[s], self.tries[s], self.swap_ready = version, False, False, 0, True
        return s

    def swap(self, force: bool = False) -> int:
        if not (self.swap_ready or force):
            raise RuntimeError("the inactive slot holds no new image")
        if self.bad[self.inactive] and not force:
            raise RuntimeError("the inactive slot is marked bad")
        self.active, self.swap_ready = self.inactive, False
        self.tries[self.active] = self.max_tries
        return self.active

    def mark_good(self, slot: Optional[int] = None) -> None:
        s = self.active if slot is None else slot
        self.good[s], self.bad[s], self.tries[s] = True, False, 0

    def mark_bad(self, slot: int) -> None:
        self.bad[slot], self.good[slot] = True, False

    def slot_is_good(self, slot: int) -> bool:
        return self.good[slot] and not self.bad[slot]

    def rollback(self) -> int:
        """Back to the other slot, which must be known good; the slot left behind is marked bad."""
        other = self.inactive
        if not self.slot_is_good(other):
            raise RuntimeError("no good slot to go back to")
        self.mark_bad(self.active)
        self.active = other
        return other

    def boot(self) -> int:
        """The slot to boot this time."""
        s = self.active
        if self.bad[s] or (not self.good[s] and self.tries[s] <= 0):
            return self.rollback()
        if not self.good[s]:
            self.tries[s] -= 1
        return s


# ------------------------------------------------------------------------------------------------ staged rollout
class CanaryRollout:
    """Rollout of a release over ``total`` units in stages (percentages of the fleet). A unit's cohort is fixed by a
    hash of its id and the release name, so the canary set only ever grows. ``promote`` moves to the next stage if
    the health gate passes (failure rate of the units that reported at this stage at most ``max_failure_rate``,
    with at least ``min_reports`` reports); ``abort`` stops the rollout and turns every unit back."""

    def __init__(self, total: int, canary: int, release: str = "release", stages: Sequence[float] = (0.25, 0.5, 1.0),
                 max_failure_rate: float = 0.05, min_reports: int = 1):
        if not 0 < canary <= total:
            raise ValueError("need 0 < canary <= total")
        first = canary / total
        self.total, self.release = total, release
        self.stages = [first] + [s for s in stages if s > first]
        if self.stages[-1] < 1.0:
            self.stages.append(1.0)
        self.stage, self.state = 0, "running"                 # running | complete | aborted
        self.max_failure_rate, self.min_reports = max_failure_rate, min_reports
        self.reports: Dict[str, bool] = {}
        self.promotions = 0

    def percentage(self) -> float:
        return 0.0 if self.state == "aborted" else 100.0 * self.stages[self.stage]

    def canary_count(self) -> int:
        return int(round(self.total * self.percentage() / 100.0))

    def _rank(self, unit_id: str) -> float:
        d = hashlib.sha256(f"{self.release}\x00{unit_id}".encode()).digest()
        return int.from_bytes(d[:8], "big") / 2 ** 64

    def is_canary(self, unit_id: str) -> bool:
        """Whether this unit runs the new release at the current stage."""
        return self.state != "aborted" and self._rank(unit_id) < self.stages[self.stage]

    def report(self, unit_id: str, healthy: bool) -> None:
        if self.is_canary(unit_id):
            self.reports[unit_id] = bool(healthy)

    def failure_rate(self) -> float:
        return 0.0 if not self.reports else sum(not h for h in self.reports.values()) / len(self.reports)

    def gate_passes(self) -> bool:
        return len(self.reports) >= self.min_reports and self.failure_rate() <= self.max_failure_rate

    def promote(self) -> bool:
        if self.state != "running" or not self.gate_passes():
            return False
        self.promotions += 1
        if self.stage + 1 == len(self.stages):
            self.state = "complete"
        else:
            self.stage += 1
            self.reports = {}
        return True

    def has_promoted(self) -> bool:
        return self.promotions > 0

    def abort(self) -> None:
        self.state = "aborted"


# ------------------------------------------------------------------------------------------------ offline bundle
class OfflineBundle:
    """One file for air-gapped installs: magic, manifest (names, sizes, hashes, metadata), optional Ed25519
    signature over the manifest, then the payloads back to back. The signature covers the hashes, so it covers the
    payloads. Layout: ``SXBUNDLE1`` | u32 manifest length | manifest JSON | u16 signature length | signature | data."""

    MAGIC = b"SXBUNDLE1"

    def __init__(self, payloads: Optional[Dict[str, bytes]] = None, meta: Optional[dict] = None):
        self.payloads: Dict[str, bytes] = dict(payloads or {})
        self.meta = dict(meta or {})
        self.signature = b""

    def _manifest(self) -> bytes:
        return canonical_json({"meta": self.meta, "files": [{"name": n, "size": len(d), "sha256": hashlib.sha256(d).hexdigest()}
                                                            for n, d in sorted(self.payloads.items())]})

    def add(self, name: str, data: bytes) -> None:
        self.payloads[name] = bytes(data)
        self.signature = b""

    def sign(self, seed: bytes) -> None:
        self.signature = crypto.ed25519_sign(seed, self._manifest())

    def is_signed(self) -> bool:
        return bool(self.signature)

    def verify(self, public_key: bytes) -> bool:
        return len(self.signature) == 64 and crypto.ed25519_verify(public_key, self._manifest(), self.signature)

    def encode(self) -> bytes:
        m = self._manifest()
        return (self.MAGIC + struct.pack(">I", len(m)) + m + struct.pack(">H", len(self.signature)) + self.signature +
                b"".join(d for _, d in sorted(self.payloads.items())))

    def size(self) -> int:
        return len(self.encode())

    @classmethod
    def decode(cls, raw: bytes) -> "OfflineBundle":
        """Parses a bundle and checks every payload against the manifest's size and hash (a signature is checked
        separately, by ``verify``, because it needs the publisher's key)."""
        n0 = len(cls.MAGIC)
        if raw[:n0] != cls.MAGIC or len(raw) < n0 + 6:
            raise ValueError("not an offline bundle")
        mlen = struct.unpack(">I", raw[n0:n0 + 4])[0]
        m = json.loads(raw[n0 + 4:n0 + 4 + mlen])
        pos = n0 + 4 + mlen
        slen = struct.unpack(">H", raw[pos:pos + 2])[0]
        sig, pos = raw[pos + 2:pos + 2 + slen], pos + 2 + slen
        b = cls(meta=m["meta"])
        for f in m["files"]:
            data = raw[pos:pos + f["size"]]
            if len(data) != f["size"] or hashlib.sha256(data).hexdigest() != f["sha256"]:
                raise ValueError(f"payload {f['name']!r} does not match the manifest")
            b.payloads[f["name"]], pos = data, pos + f["size"]
        if pos != len(raw):
            raise ValueError("trailing bytes after the last payload")
        b.signature = sig
        return b

    def save(self, path: str) -> int:
        raw = self.encode()
        with open(path, "wb") as f:
            f.write(raw)
        return len(raw)

    @classmethod
    def load(cls, path: str) -> "OfflineBundle":
        with open(path, "rb") as f:
            return cls.decode(f.read())


# ------------------------------------------------------------------------------------------------ dependency resolution
def parse_version(text: str) -> Tuple[int, int, int]:
    parts = (text.strip().lstrip("v").split("-")[0].split(".") + ["0", "0"])[:3]
    return tuple(int(p) for p in parts)          # type: ignore[return-value]


def version_matches(version: Tuple[int, int, int], constraint: str) -> bool:
    """Comma-separated clauses, all of which must hold: ``>=1.2``, ``<2``, ``==1.4.2``, ``!=1.3.0``, ``^1.2`` (same
    major, at least 1.2.0; with major 0, same minor), ``~1.2.3`` (same major.minor, at least 1.2.3), ``*``."""
    for clause in (c.strip() for c in constraint.split(",")):
        if clause in ("", "*"):
            continue
        for op in (">=", "<=", "==", "!=", ">", "<", "^", "~"):
            if clause.startswith(op):
                want = parse_version(clause[len(op):])
                break
        else:
            op, want = "==", parse_version(clause)
        ok = {">=": version >= want, "<=": version <= want, "==": version == want, "!=": version != want,
              ">": version > want, "<": version < want,
              "^": version >= want and (version[0] == want[0] if want[0] else version[:2] == want[:2]),
              "~": version >= want and version[:2] == want[:2]}[op]
        if not ok:
            return False
    return True


class DependencyConflict(RuntimeError):
    pass


class DepResolver:
    """Picks one version per package so that every constraint of every chosen version holds, preferring the newest
    versions, by depth-first search with backtracking. ``add_package`` registers what exists; ``require`` states what
    the root needs."""

    def __init__(self):
        self.available: Dict[str, Dict[Tuple[int, int, int], Dict[str, str]]] = {}
        self.roots: Dict[str, str] = {}
        self.solution: Optional[Dict[str, Tuple[int, int, int]]] = None
        self.steps = 0

    def add_package(self, name: str, version: str, deps: Optional[Dict[str, str]] = None) -> None:
        self.available.setdefault(name, {})[parse_version(version)] = dict(deps or {})
        self.solution = None

    def require(self, name: str, constraint: str = "*") -> None:
        self.roots[name] = constraint
        self.solution = None

    def reset(self) -> None:
        self.available, self.roots, self.solution, self.steps = {}, {}, None, 0

    def is_resolved(self) -> bool:
        return self.solution is not None

    def resolve(self, max_steps: int = 100000) -> Dict[str, str]:
        self.steps = 0
        picked: Dict[str, Tuple[int, int, int]] = {}
        constraints: Dict[str, List[Tuple[str, str]]] = {n: [("<root>", c)] for n, c in self.roots.items()}
        last_conflict = [""]

        def ok(name, v):
            return all(version_matches(v, c) for _, c in constraints.get(name, ()))

        def search() -> bool:
            self.steps += 1
            if self.steps > max_steps:
                raise DependencyConflict("search budget exhausted")
            for name, v in picked.items():
                if not ok(name, v):
                    last_conflict[0] = f"{name} {'.'.join(map(str, v))} violates " + \
                        ", ".join(f"{who} wants {c}" for who, c in constraints[name] if not version_matches(v, c))
                    return False
            todo = [n for n in constraints if n not in picked]
            if not todo:
                return True
            name = min(todo, key=lambda n: sum(ok(n, v) for v in self.available.get(n, {})))     # most constrained first
            if name not in self.available:
                last_conflict[0] = f"{name} is required by {constraints[name][0][0]} but no version of it is known"
                return False
            for v in sorted(self.available[name], reverse=True):
                if not ok(name, v):
                    continue
                picked[name] = v
                added = []
                for dep, c in self.available[name][v].items():
                    constraints.setdefault(dep, []).append((f"{name} {'.'.join(map(str, v))}", c))
                    added.append(dep)
                if search():
                    return True
                for dep in added:
                    constraints[dep].pop()
                    if not constraints[dep]:
                        del constraints[dep]
                        picked.pop(dep, None)
                del picked[name]
            if not last_conflict[0]:
                last_conflict[0] = f"no version of {name} satisfies " + ", ".join(f"{who}: {c}" for who, c in constraints[name])
            return False

        if not search():
            raise DependencyConflict(last_conflict[0] or "no consistent selection exists")
        self.solution = dict(picked)
        return {n: ".".join(map(str, v)) for n, v in sorted(picked.items())}

    def install_order(self) -> List[str]:
        """Dependencies before dependents (ties by name); raises on a dependency cycle."""
        if self.solution is None:
            self.resolve()
        deps = {n: sorted(d for d in self.available[n][v] if d in self.solution) for n, v in self.solution.items()}
        order, state = [], {}

        def visit(n, chain):
            if state.get(n) == 2:
                return
            if state.get(n) == 1:
                raise DependencyConflict("dependency cycle: " + " -> ".join(chain + [n]))
            state[n] = 1
            for d in deps[n]:
                visit(d, chain + [n])
            state[n] = 2
            order.append(n)

        for n in sorted(deps):
            visit(n, [])
        return order
