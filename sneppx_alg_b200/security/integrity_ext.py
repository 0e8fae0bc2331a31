"""S3 extensions: integrity baselines and host-state monitors that complement ``security/monitoring.py``.

* ``FsIntegrity``: baseline of a directory tree (hash, size, mode, owner per file) with a signed on-disk form; a scan
  reports added / removed / modified / permission-changed files; ``PersistenceMonitor`` is the same idea pointed at
  the places programs use to survive a reboot, with a reason per finding;
* ``CodeTamperDetector``: digests of registered Python functions' byte code and of the shared objects mapped into
  the process; ``MemoryMapScanner``: writable + executable anonymous mappings and code mapped from deleted files;
* ``SyscallMonitor``: sliding n-gram model of system-call sequences (unseen n-grams score as anomalies), an
  allow-list and per-call rate limits; ``TimingMonitor``: a calibrated workload whose slow-down betrays
  single-stepping or heavy instrumentation;
* ``NetConnMonitor`` (new listeners and remote peers outside the allowed networks, from ``/proc/net/tcp`` text),
  ``KernelObjectMonitor`` (module list and the kernel taint word), ``DeviceMonitor`` (devices that appear after the
  baseline);
* ``ToctouGuard``: identity token taken at check time and enforced on the opened descriptor at use time;
* ``ImaLog``: measurement list with a running aggregate (extend = hash of aggregate and entry), appraisal of files
  against reference digests, verification of a log against its aggregate;
* ``Watchdog``: the monitors' own heartbeat, so a silenced monitor is noticed.

Every reader of host state takes its input as text or through an injectable function, so the logic is testable
without the host being in a particular state. Reference behaviour: security/monitor/integrity_monitor.c and
monitor_advanced.c (function families ``fs_integrity_*``, ``code_tamper_*``, ``monitor_syscall_*``,
``monitor_timing_*``, ``net_conn_*``, ``persistence_monitor_*``, ``kernel_obj_*``, ``toctou_*``, ``ima_*``,
``device_insertion_*``, ``proc_injection_*``, ``monitor_heartbeat``).
"""
from __future__ import annotations

import fnmatch
import hashlib
import ipaddress
import json
import os
import stat
import statistics
import time
from collections import Counter, deque
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Set, Tuple

from . import crypto


def _file_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


# ------------------------------------------------------------------------------------------------ file trees
@dataclass(frozen=True)
class Change:
    kind: str           # added | removed | modified | mode | owner
    path: str
    detail: str = ""


class FsIntegrity:
    """Baseline and re-scan of the regular files under ``root`` (symbolic links are recorded by target, not
    followed). ``exclude`` holds glob patterns over root-relative paths."""

    def __init__(self, root: str, exclude: Iterable[str] = ()):
        self.root, self.exclude = os.path.abspath(root), list(exclude)
        self.baseline: Dict[str, dict] = {}

    def _walk(self) -> Dict[str, dict]:
        out = {}
        for d, dirs, files in os.walk(self.root, followlinks=False):
            for f in files:
                full = os.path.join(d, f)
                rel = os.path.relpath(full, self.root).replace(os.sep, "/")
                if any(fnmatch.fnmatch(rel, p) for p in self.exclude):
                    continue
                st = os.lstat(full)
                if stat.S_ISLNK(st.st_mode):
                    out[rel] = {"link": os.readlink(full), "mode": stat.S_IMODE(st.st_mode), "uid": st.st_uid, "gid": st.st_gid}
                elif stat.S_ISREG(st.st_mode):
                    out[rel] = {"sha256": _file_digest(full), "size": st.st_size, "mode": stat.S_IMODE(st.st_mode),
                                "uid": st.st_uid, "gid": st.st_gid}
        return out

    def snapshot(self) -> int:
        self.baseline = self._walk()
        return len(self.baseline)

    def scan(self) -> List[Change]:
        now, out = self._walk(), []
        for p in sorted(set(now) - set(self.baseline)):
            out.append(Change("added", p))
        for p in sorted(set(self.baseline) - set(now)):
            out.append(Change("removed", p))
        for p in sorted(set(now) & set(self.baseline)):
            a, b = self.baseline[p], now[p]
            if a.get("sha256") != b.get("sha256") or a.get("link") != b.get("link") or a.get("size") != b.get("size"):
                out.append(Change("modified", p))
            if a["mode"] != b["mode"]:
                out.append(Change("mode", p, f"{a['mode']:o} -> {b['mode']:o}"))
            if (a["uid"], a["gid"]) != (b["uid"], b["gid"]):
                out.append(Change("owner", p, f"{a['uid']}:{a['gid']} -> {b['uid']}:{b['gid']}"))
        return out

    def accept(self, path: Optional[str] = None) -> None:
        """Takes the current state of one file (or of everything) into the baseline."""
        now = self._walk()
        if path is None:
            self.baseline = now
        elif path in now:
            self.baseline[path] = now[path]
        else:
            self.baseline.pop(path, None)

    def save(self, path: str, signing_seed: bytes) -> None:
        body = json.dumps({"root": self.root, "exclude": self.exclude, "files": self.baseline}, sort_keys=True)
        with open(path, "w") as f:
            json.dump({"body": body, "sig": crypto.ed25519_sign(signing_seed, body.encode()).hex()}, f)

    @classmethod
    def load(cls, path: str, public_key: bytes) -> "FsIntegrity":
        with open(path) as f:
            d = json.load(f)
        if not crypto.ed25519_verify(public_key, d["body"].encode(), bytes.fromhex(d["sig"])):
            raise ValueError("baseline signature does not verify")
        body = json.loads(d["body"])
        out = cls(body["root"], body["exclude"])
        out.baseline = body["files"]
        return out


PERSISTENCE_LOCATIONS = {
    "etc/cron*/*": "scheduled job", "etc/crontab": "scheduled job", "var/spool/cron/*": "scheduled job",
    "etc/systemd/system/*": "service unit", "usr/lib/systemd/system/*": "service unit", "etc/init.d/*": "init script",
    "etc/rc.local": "init script", "etc/profile": "login shell start-up", "etc/profile.d/*": "login shell start-up",
    "etc/ld.so.preload": "library preload", "etc/ld.so.conf.d/*": "library search path",
    "root/.ssh/authorized_keys": "remote login key", "home/*/.ssh/authorized_keys": "remote login key",
    "home/*/.bashrc": "shell start-up", "root/.bashrc": "shell start-up", "etc/passwd": "account database",
    "etc/sudoers": "privilege rule", "etc/sudoers.d/*": "privilege rule", "etc/udev/rules.d/*": "device rule",
}


class PersistenceMonitor(FsIntegrity):
    """``FsIntegrity`` restricted to autostart and log-on locations under a file-system root (``/`` in production, a
    scratch tree in tests); every finding carries what the location is used for."""

    def __init__(self, root: str = "/", locations: Optional[Dict[str, str]] = None):
        super().__init__(root)
        self.locations = dict(PERSISTENCE_LOCATIONS if locations is None else locations)

    def _reason(self, rel: str) -> Optional[str]:
        return next((why for pat, why in self.locations.items() if fnmatch.fnmatch(rel, pat)), None)

    def _walk(self) -> Dict[str, dict]:
        out = {}
        tops = {p.split("/")[0] for p in self.locations}
        for top in sorted(tops):
            base = os.path.join(self.root, top)
            if not os.path.isdir(base):
                continue
            sub = FsIntegrity(base)
            for rel, rec in sub._walk().items():
                full_rel = f"{top}/{rel}"
                if self._reason(full_rel):
                    out[full_rel] = rec
        return out

    def findings(self) -> List[Tuple[Change, str]]:
        return [(c, self._reason(c.path) or "") for c in self.scan()]


# ------------------------------------------------------------------------------------------------ code in memory
class CodeTamperDetector:
    """Digests of what is supposed to stay constant while the process runs: the byte code, constants and names of
    registered functions (a monkey-patched or hot-swapped function changes them) and the on-disk bytes of shared
    objects mapped into the process."""

    def __init__(self):
        self._functions: Dict[str, Tuple[Callable[[], object], str]] = {}
        self._libraries: Dict[str, str] = {}

    @staticmethod
    def _code_digest(fn) -> str:
        code = getattr(fn, "__code__", None)
        if code is None:
            raise TypeError("only Python functions carry byte code")
        h = hashlib.sha256(code.co_code)
        h.update(repr(code.co_consts).encode())
        h.update(repr(code.co_names).encode())
        return h.hexdigest()

    def register_function(self, name: str, getter: Callable[[], object]) -> None:
        """``getter`` returns the function as it is reachable right now, e.g. ``lambda: module.handler``."""
        self._functions[name] = (getter, self._code_digest(getter()))

    def register_libraries(self, maps_text: Optional[str] = None, pattern: str = "*.so*") -> int:
        text = maps_text if maps_text is not None else open("/proc/self/maps").read()
        for path in sorted({r.path for r in parse_maps(text) if r.path.startswith("/") and fnmatch.fnmatch(os.path.basename(r.path), pattern)}):
            if os.path.isfile(path):
                self._libraries[path] = _file_digest(path)
        return len(self._libraries)

    def check(self) -> List[str]:
        bad = []
        for name, (getter, want) in self._functions.items():
            try:
                if self._code_digest(getter()) != want:
                    bad.append(f"function {name}")
            except (TypeError, AttributeError):
                bad.append(f"function {name}")
        for path, want in self._libraries.items():
            if not os.path.isfile(path) or _file_digest(path) != want:
                bad.append(f"library {path}")
        return bad


@dataclass(frozen=True)
class MapRegion:
    start: int
    end: int
    perms: str
    path: str


def parse_maps(text: str) -> List[MapRegion]:
    """Regions of a ``/proc/<pid>/maps`` listing."""
    out = []
    for line in text.splitlines():
        parts = line.split(None, 5)
        if len(parts) < 5 or "-" not in parts[0]:
            continue
        a, b = parts[0].split("-")
        out.append(MapRegion(int(a, 16), int(b, 16), parts[1], parts[5].strip() if len(parts) > 5 else ""))
    return out


class MemoryMapScanner:
    """Signs of code injection in an address-space listing: mappings that are writable and executable at once
    (outside an allow-list of names such as a JIT's), executable anonymous memory, executable mappings whose file has
    been deleted."""

    def __init__(self, allow: Iterable[str] = ("[vdso]", "[vsyscall]")):
        self.allow = set(allow)

    def scan(self, maps_text: Optional[str] = None) -> List[Tuple[str, MapRegion]]:
        text = maps_text if maps_text is not None else open("/proc/self/maps").read()
        out = []
        for r in parse_maps(text):
            if "x" not in r.perms or r.path in self.allow:
                continue
            if "w" in r.perms:
                out.append(("writable and executable", r))
            elif r.path == "" or r.path.startswith("[anon"):
                out.append(("executable anonymous memory", r))
            elif r.path.endswith(" (deleted)"):
                out.append(("code from a deleted file", r))
        return out


# ------------------------------------------------------------------------------------------------ behaviour
class SyscallMonitor:
    """Sequence model in the manner of stide (Forrest et al.): every window of ``n`` consecutive calls seen in
    training is normal; the anomaly score of a trace is the share of its windows that were never seen. On top of
    that: calls outside ``allowed`` are violations outright, and ``limits`` caps calls per ``window_s`` seconds."""

    def __init__(self, n: int = 3, allowed: Optional[Iterable[str]] = None, limits: Optional[Dict[str, int]] = None,
                 window_s: float = 1.0, clock: Callable[[], float] = time.monotonic):
        self.n, self.allowed, self.limits, self.window_s, self.clock = n, (set(allowed) if allowed is not None else None), \
            dict(limits or {}), window_s, clock
        self.normal: Set[Tuple[str, ...]] = set()
        self._recent: deque = deque(maxlen=n)
        self._times: Dict[str, deque] = {}
        self.counts: Counter = Counter()
        self.violations: List[Tuple[str, str]] = []

    def _windows(self, seq: Sequence[str]):
        return (tuple(seq[i:i + self.n]) for i in range(len(seq) - self.n + 1))

    def train(self, traces: Iterable[Sequence[str]]) -> int:
        for t in traces:
            self.normal.update(self._windows(list(t)))
        return len(self.normal)

    def score(self, trace: Sequence[str]) -> float:
        w = list(self._windows(list(trace)))
        return sum(x not in self.normal for x in w) / len(w) if w else 0.0

    def observe(self, call: str) -> List[str]:
        """Feeds one live call; returns the reasons it is suspicious (empty when it is not)."""
        why = []
        self.counts[call] += 1
        if self.allowed is not None and call not in self.allowed:
            why.append("not in the allow-list")
        if call in self.limits:
            now = self.clock()
            q = self._times.setdefault(call, deque())
            q.append(now)
            while q and now - q[0] > self.window_s:
                q.popleft()
            if len(q) > self.limits[call]:
                why.append(f"more than {self.limits[call]} per {self.window_s:g}s")
        self._recent.append(call)
        if self.normal and len(self._recent) == self.n and tuple(self._recent) not in self.normal:
            why.append("unseen sequence " + " > ".join(self._recent))
        self.violations += [(call, w) for w in why]
        return why

    def frequency(self) -> Dict[str, float]:
        total = sum(self.counts.values())
        return {k: v / total for k, v in self.counts.most_common()} if total else {}


class TimingMonitor:
    """Runs a fixed workload, remembers how long it takes (median of ``calibration_runs``) and later reports when a
    run takes ``threshold`` times as long: a debugger single-stepping the process, or instrumentation, shows up as a
    large constant factor, scheduling noise does not."""

    def __init__(self, workload: Optional[Callable[[], None]] = None, threshold: float = 8.0, calibration_runs: int = 9,
                 clock: Callable[[], float] = time.perf_counter):
        self.workload = workload or self._default
        self.threshold, self.calibration_runs, self.clock = threshold, calibration_runs, clock
        self.reference: Optional[float] = None
        self.history: List[float] = []

    @staticmethod
    def _default() -> None:
        x = 0
        for i in range(20000):
            x = (x * 31 + i) & 0xFFFFFFFF

    def _time(self) -> float:
        t0 = self.clock()
        self.workload()
        return self.clock() - t0

    def calibrate(self) -> float:
        self.reference = statistics.median(self._time() for _ in range(self.calibration_runs))
        return self.reference

    def check(self, runs: int = 3) -> Tuple[bool, float]:
        """(suspicious, slow-down factor): the fastest of ``runs`` runs against the calibrated reference."""
        if self.reference is None:
            self.calibrate()
        best = min(self._time() for _ in range(runs))
        ratio = best / max(self.reference, 1e-12)
        self.history.append(ratio)
        return ratio >= self.threshold, ratio


# ------------------------------------------------------------------------------------------------ host state
_TCP_STATES = {"01": "ESTABLISHED", "02": "SYN_SENT", "03": "SYN_RECV", "04": "FIN_WAIT1", "05": "FIN_WAIT2", "06": "TIME_WAIT",
               "07": "CLOSE", "08": "CLOSE_WAIT", "09": "LAST_ACK", "0A": "LISTEN", "0B": "CLOSING"}


def _proc_addr(text: str) -> Tuple[str, int]:
    host, port = text.split(":")
    raw = bytes.fromhex(host)
    if len(raw) == 4:
        return str(ipaddress.IPv4Address(raw[::-1])), int(port, 16)
    words = b"".join(raw[i:i + 4][::-1] for i in range(0, 16, 4))          # four little-endian 32-bit words
    return str(ipaddress.IPv6Address(words)), int(port, 16)


def parse_proc_net_tcp(text: str) -> List[dict]:
    """Sockets of a ``/proc/net/tcp`` or ``/proc/net/tcp6`` listing: local / remote address and port, state, uid."""
    out = []
    for line in text.splitlines()[1:]:
        p = line.split()
        if len(p) < 8 or ":" not in p[1]:
            continue
        (la, lp), (ra, rp) = _proc_addr(p[1]), _proc_addr(p[2])
        out.append({"local": la, "local_port": lp, "remote": ra, "remote_port": rp, "state": _TCP_STATES.get(p[3], p[3]), "uid": int(p[7])})
    return out


class NetConnMonitor:
    """Compares the socket table with a baseline of listening ports and a list of networks the process is allowed to
    talk to. Findings: a port that was not listening at baseline time, an established connection to a peer outside
    the allowed networks."""

    def __init__(self, allowed_networks: Iterable[str] = ("127.0.0.0/8", "::1/128"), reader: Optional[Callable[[], str]] = None):
        self.allowed = [ipaddress.ip_network(n) for n in allowed_networks]
        self.reader = reader or (lambda: open("/proc/net/tcp").read())
        self.listeners: Set[int] = set()

    def baseline(self) -> Set[int]:
        self.listeners = {s["local_port"] for s in parse_proc_net_tcp(self.reader()) if s["state"] == "LISTEN"}
        return set(self.listeners)

    def _allowed(self, addr: str) -> bool:
        ip = ipaddress.ip_address(addr)
        if ip.version == 6 and ip.ipv4_mapped is not None:
            ip = ip.ipv4_mapped
        return any(ip.version == n.version and ip in n for n in self.allowed)

    def scan(self) -> List[Tuple[str, dict]]:
        out = []
        for s in parse_proc_net_tcp(self.reader()):
            if s["state"] == "LISTEN" and s["local_port"] not in self.listeners:
                out.append(("new listener", s))
            elif s["state"] == "ESTABLISHED" and not self._allowed(s["remote"]):
                out.append(("peer outside the allowed networks", s))
        return out


class KernelObjectMonitor:
    """Loaded kernel modules (``/proc/modules`` text) against a baseline, and the kernel's taint word decoded into
    its flags (out-of-tree module, unsigned module, forced load ...)."""

    TAINT_FLAGS = {0: "proprietary module", 1: "module force-loaded", 2: "kernel out of specification", 3: "module force-unloaded",
                   4: "machine check", 5: "bad page", 6: "taint requested by user space", 7: "kernel died recently",
                   8: "ACPI table overridden", 9: "kernel warning", 10: "staging driver", 11: "firmware workaround",
                   12: "out-of-tree module", 13: "unsigned module", 14: "soft lockup", 15: "live patched"}

    def __init__(self, modules_reader: Optional[Callable[[], str]] = None, taint_reader: Optional[Callable[[], str]] = None):
        self.modules_reader = modules_reader or (lambda: open("/proc/modules").read())
        self.taint_reader = taint_reader or (lambda: open("/proc/sys/kernel/tainted").read())
        self.modules: Set[str] = set()

    def _current(self) -> Set[str]:
        return {l.split()[0] for l in self.modules_reader().splitlines() if l.strip()}

    def baseline(self) -> int:
        self.modules = self._current()
        return len(self.modules)

    def scan(self) -> Dict[str, List[str]]:
        now = self._current()
        return {"loaded": sorted(now - self.modules), "unloaded": sorted(self.modules - now)}

    def taint(self) -> List[str]:
        word = int(self.taint_reader().strip() or 0)
        return [name for bit, name in self.TAINT_FLAGS.items() if word >> bit & 1]


class DeviceMonitor:
    """Devices (any listing of identifiers: USB bus entries, block devices, PCI functions) that appear or vanish after
    the baseline."""

    def __init__(self, lister: Optional[Callable[[], Iterable[str]]] = None):
        self.lister = lister or (lambda: os.listdir("/sys/bus/usb/devices") if os.path.isdir("/sys/bus/usb/devices") else [])
        self.known: Set[str] = set()

    def baseline(self) -> int:
        self.known = set(self.lister())
        return len(self.known)

    def scan(self) -> Dict[str, List[str]]:
        now = set(self.lister())
        return {"inserted": sorted(now - self.known), "removed": sorted(self.known - now)}


# ------------------------------------------------------------------------------------------------ check / use
class ToctouError(RuntimeError):
    pass


class ToctouGuard:
    """Closes the gap between checking a file and using it: ``check`` records the file's identity (device, inode,
    size, modification time, optionally its digest); ``open_verified`` opens without following a final symbolic link
    and compares the identity of the descriptor it got with the recorded one, so a file swapped in between is
    refused."""

    def __init__(self, with_digest: bool = False):
        self.with_digest = with_digest
        self.checks = self.mismatches = 0

    def check(self, path: str) -> dict:
        st = os.lstat(path)
        if not stat.S_ISREG(st.st_mode):
            raise ToctouError("not a regular file")
        self.checks += 1
        tok = {"path": path, "dev": st.st_dev, "ino": st.st_ino, "size": st.st_size, "mtime_ns": st.st_mtime_ns}
        if self.with_digest:
            tok["sha256"] = _file_digest(path)
        return tok

    def open_verified(self, token: dict, mode: str = "rb"):
        fd = os.open(token["path"], os.O_RDONLY | getattr(os, "O_NOFOLLOW", 0))
        try:
            st = os.fstat(fd)
            same = (st.st_dev, st.st_ino, st.st_size, st.st_mtime_ns) == (token["dev"], token["ino"], token["size"], token["mtime_ns"])
            if same and "sha256" in token:
                h, off = hashlib.sha256(), 0
                while True:
                    chunk = os.pread(fd, 1 << 20, off)         # positional reads: the descriptor's offset stays at 0
                    if not chunk:
                        break
                    h.update(chunk)
                    off += len(chunk)
                same = h.hexdigest() == token["sha256"]
            f = os.fdopen(fd, mode)
        except Exception:
            os.close(fd)
            raise
        if not same:
            f.close()
            self.mismatches += 1
            raise ToctouError(f"{token['path']} changed between check and use")
        return f


# ------------------------------------------------------------------------------------------------ measurement log
class ImaLog:
    """Measurement list in the manner of the kernel's integrity measurement architecture: each measured file adds an
    entry (digest, path) and extends the aggregate, ``aggregate = SHA-256(aggregate || SHA-256(digest || path))``, so
    the aggregate commits to the whole ordered list. ``appraise`` compares a file with a reference digest before it
    is used; ``verify`` replays a list against an aggregate (for instance one quoted by a TPM)."""

    def __init__(self):
        self.entries: List[Tuple[str, str]] = []
        self.aggregate = b"\0" * 32
        self._seen: Set[Tuple[str, str]] = set()

    @staticmethod
    def _extend(aggregate: bytes, digest: str, path: str) -> bytes:
        return hashlib.sha256(aggregate + hashlib.sha256(bytes.fromhex(digest) + path.encode()).digest()).digest()

    def measure(self, path: str, data: Optional[bytes] = None) -> str:
        """Measures a file (or the given bytes under that name). The same content under the same path is measured
        once, as IMA does."""
        digest = hashlib.sha256(data).hexdigest() if data is not None else _file_digest(path)
        if (digest, path) not in self._seen:
            self._seen.add((digest, path))
            self.entries.append((digest, path))
            self.aggregate = self._extend(self.aggregate, digest, path)
        return digest

    def appraise(self, path: str, reference: Dict[str, str], data: Optional[bytes] = None) -> bool:
        """True when the file's digest equals the reference digest for its path; the file is measured either way."""
        return reference.get(path) == self.measure(path, data)

    @classmethod
    def verify(cls, entries: Iterable[Tuple[str, str]], aggregate: bytes) -> bool:
        agg = b"\0" * 32
        for digest, path in entries:
            agg = cls._extend(agg, digest, path)
        return agg == aggregate

    def export(self) -> str:
        return "\n".join(f"{d} {p}" for d, p in self.entries) + ("\n" if self.entries else "")

    def measurement_count(self) -> int:
        return len(self.entries)


# ------------------------------------------------------------------------------------------------ monitor heartbeat
class Watchdog:
    """Heartbeats of the monitors themselves: each registered monitor promises a beat every ``interval_s``;
    ``missed`` lists those that have been silent for longer than ``grace`` intervals."""

    def __init__(self, grace: float = 2.0, clock: Callable[[], float] = time.monotonic):
        self.grace, self.clock = grace, clock
        self._monitors: Dict[str, Tuple[float, float]] = {}            # name -> (interval, last beat)
        self.beats: Counter = Counter()

    def register(self, name: str, interval_s: float) -> None:
        self._monitors[name] = (float(interval_s), self.clock())

    def unregister(self, name: str) -> bool:
        return self._monitors.pop(name, None) is not None

    def heartbeat(self, name: str) -> None:
        if name not in self._monitors:
            raise KeyError(name)
        self._monitors[name] = (self._monitors[name][0], self.clock())
        self.beats[name] += 1

    def missed(self) -> List[str]:
        now = self.clock()
        return sorted(n for n, (iv, last) in self._monitors.items() if now - last > self.grace * iv)

    def status(self) -> Dict[str, dict]:
        now = self.clock()
        return {n: {"interval_s": iv, "silent_s": now - last, "beats": self.beats[n], "ok": now - last <= self.grace * iv}
                for n, (iv, last) in sorted(self._monitors.items())}
