"""S7 extensions (``security/updates_ext.py``): TUF metadata workflow and its attack checks, BSDIFF40 deltas, signed
manifests, the software TPM, A/B slots, canary rollout, offline bundles, dependency resolution."""
import bz2
import copy
import hashlib
import os
import random

import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security import updates_ext as ux


def test_tuf_workflow_rotation_and_attacks():
    now = [1_000_000.0]
    repo = ux.TufRepository(thresholds={"root": 2}, keys_per_role={"root": 3}, clock=lambda: now[0])
    repo.add_target("model.bin", b"weights v1")
    repo.publish()
    client = ux.TufClient(repo.fetch("root", 1), clock=lambda: now[0])
    assert client.refresh(repo) == {"root": 1, "targets": 2, "snapshot": 2, "timestamp": 2}
    assert client.download(repo, "model.bin") == b"weights v1" and client.target_info("other") is None
    # a changed target file is refused; an unlisted one too
    repo.targets["model.bin"] = b"weights v1 (tampered)"
    with pytest.raises(ux.TufError, match="length or hash"):
        client.download(repo, "model.bin")
    with pytest.raises(ux.TufError, match="not a trusted target"):
        client.download(repo, "extra.bin")
    repo.targets["model.bin"] = b"weights v1"
    # rollback: the repository serves older (validly signed) timestamp metadata
    old = copy.deepcopy(repo.metadata)
    repo.add_target("model.bin", b"weights v2")
    repo.publish()
    client.refresh(repo)
    newer = copy.deepcopy(repo.metadata)
    repo.metadata = old
    with pytest.raises(ux.TufError, match="went back"):
        client.refresh(repo)
    # mix and match: new timestamp + snapshot with the old targets file
    repo.metadata = dict(newer, targets=old["targets"])
    with pytest.raises(ux.TufError, match="targets"):
        client.refresh(repo)
    repo.metadata = newer
    # a forged targets file signed by a key the root does not list
    forged = ux._sign_metadata(dict(newer["targets"]["signed"], targets={}), [os.urandom(32)])
    repo.metadata = dict(newer, targets=forged)
    with pytest.raises(ux.TufError, match="0 valid signatures"):
        client.refresh(repo)
    repo.metadata = newer
    # freeze: nothing new is published and the timestamp runs out
    now[0] += 2 * 86400.0
    with pytest.raises(ux.TufError, match="timestamp: metadata has expired"):
        client.refresh(repo)
    repo.refresh_timestamp()
    assert client.refresh(repo)["timestamp"] == repo.versions["timestamp"]
    # key rotation: an online key, then one of the root keys; a client that was offline walks the whole chain
    repo.rotate_key("timestamp")
    repo.rotate_key("root", 1)
    assert client.refresh(repo)["root"] == 3 and client.download(repo, "model.bin") == b"weights v2"
    fresh = ux.TufClient(repo.fetch("root", 1), clock=lambda: now[0])
    assert fresh.refresh(repo)["root"] == 3
    # a root signed by one key only does not meet the threshold of two
    lone = ux._sign_metadata(repo.metadata["root"]["signed"], repo.seeds["root"][:1])
    with pytest.raises(ux.TufError, match="1 valid signatures, threshold 2"):
        ux.TufClient(lone)
    # the same signature listed twice counts once
    dup = dict(lone, signatures=lone["signatures"] * 2)
    with pytest.raises(ux.TufError, match="1 valid signatures"):
        ux.TufClient(dup)
    assert repo.remove_target("model.bin") and not repo.remove_target("model.bin")


def test_bsdiff_patches_round_trip_and_stay_small():
    rng = random.Random(0)
    old = os.urandom(30000)
    new = bytearray(old[:7000] + os.urandom(400) + old[7000:18000] + old[22000:])
    for i in rng.sample(range(len(new)), 300):
        new[i] ^= 1 << rng.randrange(8)
    new = bytes(new)
    patch = ux.bsdiff(old, new)
    assert patch[:8] == b"BSDIFF40" and ux.bsdiff_total_size(patch) == len(new) and ux.bspatch(old, patch) == new
    assert len(patch) < 2500 < len(bz2.compress(new))                          # far smaller than shipping the file
    for a, b in ((b"", b""), (b"abc", b""), (b"", b"abc"), (b"same" * 50, b"same" * 50), (old[:2000], old[:2000][::-1]),
                 (b"A" * 1000, b"A" * 400 + b"B" + b"A" * 700)):
        assert ux.bspatch(a, ux.bsdiff(a, b)) == b
    # a patch in the original tool's layout applies: one control triple (diff 3, extra 2, seek 0)
    ctrl = ux._offtout(3) + ux._offtout(2) + ux._offtout(0)
    cz, dz, ez = bz2.compress(ctrl), bz2.compress(bytes([1, 0, 255])), bz2.compress(b"XY")
    hand = b"BSDIFF40" + ux._offtout(len(cz)) + ux._offtout(len(dz)) + ux._offtout(5) + cz + dz + ez
    assert ux.bspatch(b"abc", hand) == b"bbbXY" and ux._offtin(ux._offtout(-5)) == -5
    with pytest.raises(ValueError):
        ux.bspatch(old, b"BSDIFF41" + patch[8:])
    with pytest.raises(ValueError):
        ux.bspatch(old, patch[:24] + ux._offtout(len(new) + 1) + patch[32:])
    seed = os.urandom(32)
    p, sig = ux.bsdiff_signed(old, new, seed)
    pub = crypto.ed25519_public_key(seed)
    assert ux.bspatch_verified(old, p, sig, pub) == new
    with pytest.raises(ValueError, match="signature"):
        ux.bspatch_verified(old[:-1] + b"x", p, sig, pub)                        # right patch, wrong starting file


def test_bsdiff_files_and_manifest(tmp_path):
    rel = tmp_path / "release"
    (rel / "bin").mkdir(parents=True)
    (rel / "bin" / "tool").write_bytes(b"\x7fELF" + os.urandom(500))
    (rel / "README").write_text("hello")
    (tmp_path / "old").write_bytes(b"version one " * 100)
    (tmp_path / "new").write_bytes(b"version one " * 60 + b"version two " * 40)
    n = ux.bsdiff_files(str(tmp_path / "old"), str(tmp_path / "new"), str(tmp_path / "p"))
    assert n == (tmp_path / "p").stat().st_size and ux.bspatch_files(str(tmp_path / "old"), str(tmp_path / "p"), str(tmp_path / "out")) == 1200
    assert (tmp_path / "out").read_bytes() == (tmp_path / "new").read_bytes()
    m = ux.Manifest.create(str(rel), meta={"version": "1.2.0"})
    assert sorted(m.files) == ["README", "bin/tool"] and m.files["README"]["sha256"] == hashlib.sha256(b"hello").hexdigest()
    seed = os.urandom(32)
    sig, pub = m.sign(seed), crypto.ed25519_public_key(seed)
    back = ux.Manifest.decode(m.encode())
    assert back.digest() == m.digest() and back.verify(sig, pub) and back.verify_all(str(rel), sig, pub)
    (rel / "README").write_text("hellO")
    (rel / "stray").write_text("x")
    assert back.check_files(str(rel)) == ["hash: README", "unlisted: stray"] and not back.verify_all(str(rel), sig, pub)
    (rel / "README").write_text("hello, longer")
    os.remove(rel / "bin" / "tool")
    assert back.check_files(str(rel)) == ["missing: bin/tool", "size: README", "unlisted: stray"]
    back.meta["version"] = "9.9.9"
    assert not back.verify(sig, pub)
    with pytest.raises(ValueError):
        ux.Manifest.create(str(rel), ["../old"])


def test_soft_tpm_quotes_and_sealing():
    tpm = ux.SoftTpm(b"e" * 32)
    assert tpm.pcr_read(0) == b"\0" * 32
    v1 = tpm.measure(0, b"bootloader", "stage 1")
    assert v1 == hashlib.sha256(b"\0" * 32 + hashlib.sha256(b"bootloader").digest()).digest()
    tpm.measure(0, b"kernel", "stage 2")
    tpm.measure(7, b"secure-boot-policy")
    assert ux.SoftTpm.replay_log(tpm.log) == {0: tpm.pcr_read(0), 7: tpm.pcr_read(7)}
    mask = (1 << 0) | (1 << 7)
    q = tpm.quote(b"nonce-1", mask)
    pub = tpm.attestation_public
    assert ux.SoftTpm.verify_quote(q, pub, b"nonce-1") and not ux.SoftTpm.verify_quote(q, pub, b"nonce-2")
    assert ux.SoftTpm.verify_quote(q, pub, b"nonce-1", {0: tpm.pcr_read(0), 7: tpm.pcr_read(7)})
    assert not ux.SoftTpm.verify_quote(q, pub, b"nonce-1", {0: v1, 7: tpm.pcr_read(7)})
    assert not ux.SoftTpm.verify_quote(q, pub, b"nonce-1", {0: tpm.pcr_read(0)})
    assert not ux.SoftTpm.verify_quote(q, ux.SoftTpm(b"f" * 32).attestation_public, b"nonce-1")
    sealed = tpm.seal(b"disk key", mask)
    assert tpm.unseal(sealed) == b"disk key"
    tpm.measure(3, b"unrelated")
    assert tpm.unseal(sealed) == b"disk key"                                    # PCR 3 is not in the selection
    tpm.measure(7, b"tampered policy")
    with pytest.raises(ux.TpmError, match="PCR state differs"):
        tpm.unseal(sealed)
    same_boot = ux.SoftTpm(b"e" * 32)
    for data, idx in ((b"bootloader", 0), (b"kernel", 0), (b"secure-boot-policy", 7)):
        same_boot.measure(idx, data)
    assert same_boot.unseal(sealed) == b"disk key"                               # same device, same measurements: opens again
    with pytest.raises(ux.TpmError):
        ux.SoftTpm(b"g" * 32).unseal(sealed)                                    # another device
    for bad in (lambda: tpm.extend(24, b"\0" * 32), lambda: tpm.extend(0, b"short"), lambda: tpm.quote(b"n", 0)):
        with pytest.raises(ux.TpmError):
            bad()
    tpm.set_variable(2, 2 ** 32 + 5)
    assert tpm.get_variable(2) == 5 and tpm.get_variable(9) == 0
    tpm.reset()
    assert tpm.pcr_read(0) == b"\0" * 32 and tpm.log == []


def test_ab_slots_fall_back_after_failed_boots():
    ab = ux.ABPartition(max_tries=2)
    assert ab.active == 0 and ab.boot() == 0
    with pytest.raises(RuntimeError):
        ab.swap()
    assert ab.write_inactive("2.0") == 1 and ab.swap_ready and ab.swap() == 1 and not ab.slot_is_good(1)
    assert [ab.boot(), ab.boot()] == [1, 1]                                      # two attempts, never marked good
    assert ab.boot() == 0 and ab.active == 0 and ab.bad[1] and ab.slot_is_good(0)  # fell back, new slot marked bad
    ab.write_inactive("2.1")
    ab.swap()
    assert ab.boot() == 1
    ab.mark_good()
    assert [ab.boot() for _ in range(5)] == [1] * 5 and ab.slot_is_good(1) and ab.versions == ["", "2.1"]
    assert ab.rollback() == 0 and ab.bad[1]
    ab.mark_bad(1)
    with pytest.raises(RuntimeError, match="no good slot"):
        ab.rollback()
    with pytest.raises(RuntimeError, match="marked bad"):
        ab.swap_ready = True
        ab.swap()
    assert ab.swap(force=True) == 1


def test_canary_rollout_stages_and_gate():
    ro = ux.CanaryRollout(total=1000, canary=50, release="v2", stages=(0.25, 0.5, 1.0), max_failure_rate=0.1, min_reports=5)
    units = [f"node-{i}" for i in range(1000)]
    first = {u for u in units if ro.is_canary(u)}
    assert ro.percentage() == 5.0 and ro.canary_count() == 50 and 25 <= len(first) <= 80 and not ro.promote()
    for u in first:
        ro.report(u, True)
    ro.report("node-not-canary-xyz", False)
    assert ro.gate_passes() and ro.promote() and ro.percentage() == 25.0 and ro.has_promoted()
    second = {u for u in units if ro.is_canary(u)}
    assert first < second and 190 <= len(second) <= 310                         # the cohort only grows
    for i, u in enumerate(sorted(second)):
        ro.report(u, i % 5 != 0)                                                 # 20 % failures
    assert ro.failure_rate() == pytest.approx(0.2, abs=0.01) and not ro.promote() and ro.percentage() == 25.0
    for u in second:
        ro.report(u, True)
    assert ro.promote() and ro.percentage() == 50.0
    other = ux.CanaryRollout(1000, 50, release="v3")
    assert {u for u in units if other.is_canary(u)} != first                     # another release draws another cohort
    ro.abort()
    assert ro.percentage() == 0.0 and not ro.is_canary(sorted(first)[0]) and not ro.promote()
    done = ux.CanaryRollout(10, 10)
    done.report("a", True)
    assert done.percentage() == 100.0 and done.promote() and done.state == "complete" and not done.promote()
    with pytest.raises(ValueError):
        ux.CanaryRollout(10, 0)


def test_offline_bundle(tmp_path):
    seed = os.urandom(32)
    pub = crypto.ed25519_public_key(seed)
    b = ux.OfflineBundle({"model.bin": os.urandom(3000), "config.json": b"{}"}, meta={"version": "3.1"})
    assert not b.is_signed() and not b.verify(pub)
    b.sign(seed)
    n = b.save(str(tmp_path / "u.bundle"))
    assert n == b.size() and b.is_signed()
    back = ux.OfflineBundle.load(str(tmp_path / "u.bundle"))
    assert back.verify(pub) and back.payloads == b.payloads and back.meta == {"version": "3.1"}
    assert not back.verify(crypto.ed25519_public_key(os.urandom(32)))
    raw = bytearray(b.encode())
    raw[-10] ^= 1
    with pytest.raises(ValueError, match="does not match the manifest"):
        ux.OfflineBundle.decode(bytes(raw))
    with pytest.raises(ValueError, match="trailing"):
        ux.OfflineBundle.decode(b.encode() + b"x")
    with pytest.raises(ValueError, match="not an offline bundle"):
        ux.OfflineBundle.decode(b"garbage")
    back.add("late.txt", b"x")
    assert not back.is_signed()                                                  # adding a payload voids the signature
    swapped = ux.OfflineBundle(dict(b.payloads, **{"config.json": b"{ }"}), meta=b.meta)
    swapped.signature = b.signature
    assert not swapped.verify(pub)


def test_dependency_resolution():
    assert ux.parse_version("v1.2") == (1, 2, 0) and ux.parse_version("2.0.1-rc1") == (2, 0, 1)
    vm = ux.version_matches
    assert vm((1, 4, 2), ">=1.2,<2") and not vm((2, 0, 0), ">=1.2,<2") and vm((1, 4, 2), "^1.2") and not vm((2, 0, 0), "^1.2")
    assert vm((0, 3, 9), "^0.3.1") and not vm((0, 4, 0), "^0.3.1") and vm((1, 2, 9), "~1.2.3") and not vm((1, 3, 0), "~1.2.3")
    assert vm((1, 0, 0), "*") and vm((1, 0, 0), "1.0.0") and not vm((1, 0, 0), "!=1.0.0")
    r = ux.DepResolver()
    r.add_package("app", "1.0.0", {"web": "^2.0", "db": ">=1.0"})
    for v, deps in (("2.0.0", {"json": "^1.0"}), ("2.1.0", {"json": "^2.0"})):
        r.add_package("web", v, deps)
    for v, deps in (("1.0.0", {"json": "^1.0"}), ("1.5.0", {"json": "^1.2"})):
        r.add_package("db", v, deps)
    for v in ("1.0.0", "1.2.0", "1.3.0", "2.0.0"):
        r.add_package("json", v)
    r.require("app")
    # the newest web (2.1.0) wants json 2.x, which no db accepts: the resolver has to back off to web 2.0.0
    assert r.resolve() == {"app": "1.0.0", "db": "1.5.0", "json": "1.3.0", "web": "2.0.0"} and r.is_resolved()
    order = r.install_order()
    assert order.index("json") < order.index("db") < order.index("app") and order.index("web") < order.index("app")
    r.require("json", "^2.0")
    with pytest.raises(ux.DependencyConflict):
        r.resolve()
    assert not r.is_resolved()
    r.reset()
    r.add_package("a", "1.0.0", {"ghost": "*"})
    r.require("a")
    with pytest.raises(ux.DependencyConflict, match="ghost is required by a 1.0.0"):
        r.resolve()
    r.reset()
    r.add_package("x", "1.0.0", {"y": "*"})
    r.add_package("y", "1.0.0", {"x": "*"})
    r.require("x")
    assert r.resolve() == {"x": "1.0.0", "y": "1.0.0"}
    with pytest.raises(ux.DependencyConflict, match="cycle"):
        r.install_order()
