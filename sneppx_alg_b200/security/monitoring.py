"""S3 monitoring extensions: container-breakout detection, function-table watching, metric anomaly detection and an
event correlator.

``BreakoutDetector`` consumes process events (namespace changes, mounts, capability sets, sensitive file access,
system calls) and classifies them against container-escape rules: entering the host's namespaces, mounting the
host's devices / proc / cgroup control files, gaining CAP_SYS_ADMIN-class capabilities, touching the container
runtime's sockets or release_agent, calling module-loading / ptrace-class system calls. ``FunctionTableWatch`` keeps
a digest of a dispatch table (name -> callable) and reports replaced entries. ``AnomalyDetector`` is an exponentially
weighted mean / variance per metric with a z-score alarm and a warm-up period. ``EventCorrelator`` raises a combined
alert when several different detectors fire for the same subject within a time window.
Reference modules of the same purpose: security/monitor/container_breakout.c (detect_ns_change / detect_mount /
detect_capability / check_file_access / detect_syscall / watch files / stats), security/monitor/monitor_advanced.c
(function-pointer detector, ML anomaly detector) and security/monitor/integrity_monitor.c.
"""
from __future__ import annotations

import fnmatch
import math
import time
from collections import defaultdict, deque
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Tuple

CAP_BITS = {"CAP_DAC_OVERRIDE": 1, "CAP_DAC_READ_SEARCH": 2, "CAP_NET_ADMIN": 12, "CAP_NET_RAW": 13, "CAP_SYS_MODULE": 16,
            "CAP_SYS_RAWIO": 17, "CAP_SYS_CHROOT": 18, "CAP_SYS_PTRACE": 19, "CAP_SYS_ADMIN": 21, "CAP_SYS_BOOT": 22,
            "CAP_MKNOD": 27, "CAP_BPF": 39}
DANGEROUS_CAPS = ("CAP_SYS_ADMIN", "CAP_SYS_MODULE", "CAP_SYS_PTRACE", "CAP_SYS_RAWIO", "CAP_DAC_READ_SEARCH", "CAP_BPF")
DANGEROUS_SYSCALLS = {"init_module": 0.9, "finit_module": 0.9, "delete_module": 0.7, "ptrace": 0.6, "process_vm_writev": 0.7,
                      "setns": 0.8, "unshare": 0.5, "mount": 0.6, "pivot_root": 0.8, "kexec_load": 1.0, "bpf": 0.5,
                      "open_by_handle_at": 0.9, "keyctl": 0.4, "userfaultfd": 0.4}
SENSITIVE_PATHS = ["/var/run/docker.sock", "/run/containerd/containerd.sock", "/run/crio/crio.sock", "/proc/sys/kernel/core_pattern",
                   "/proc/sysrq-trigger", "/proc/kcore", "/sys/fs/cgroup/*/release_agent", "/sys/kernel/uevent_helper",
                   "/dev/mem", "/dev/kmem", "/dev/sd*", "/dev/nvme*", "/etc/shadow", "/host/*", "/proc/1/root/*"]
HOST_MOUNT_SOURCES = ("/dev/", "proc", "sysfs", "cgroup", "/var/run/docker.sock", "/")


@dataclass
class Alert:
    kind: str
    severity: float
    pid: int
    comm: str
    detail: str
    time: float = 0.0


class BreakoutDetector:
    def __init__(self, clock: Callable[[], float] = time.time, allow_comms: Iterable[str] = ("runc", "containerd-shim")):
        self.clock = clock
        self.allow = set(allow_comms)
        self.baseline_ns: Dict[int, Dict[str, int]] = {}
        self.watch = list(SENSITIVE_PATHS)
        self.alerts: List[Alert] = []
        self.counts = defaultdict(int)

    def _raise(self, kind, sev, pid, comm, detail) -> Optional[Alert]:
        self.counts["events"] += 1
        if comm in self.allow:
            self.counts["allowed"] += 1
            return None
        a = Alert(kind, sev, pid, comm, detail, self.clock())
        self.alerts.append(a)
        self.counts[kind] += 1
        return a

    def record_namespaces(self, pid: int, ns: Dict[str, int]) -> None:
        """Inode numbers of a process's namespaces (``/proc/<pid>/ns/*``) at container start."""
        self.baseline_ns[pid] = dict(ns)

    def detect_ns_change(self, pid: int, ns: Dict[str, int], comm: str = "", host_ns: Optional[Dict[str, int]] = None):
        base = self.baseline_ns.get(pid)
        if base is None:
            self.baseline_ns[pid] = dict(ns)
            return None
        changed = [k for k in ns if base.get(k) != ns[k]]
        if not changed:
            self.counts["events"] += 1
            return None
        to_host = host_ns is not None and any(ns[k] == host_ns.get(k) for k in changed)
        self.baseline_ns[pid] = dict(ns)
        return self._raise("namespace_change", 1.0 if to_host else 0.6, pid, comm,
                           f"{','.join(changed)} changed" + (" to the host's namespace" if to_host else ""))

    def detect_mount(self, pid: int, source: str, target: str, comm: str = "", fstype: str = ""):
        risky = fstype in ("proc", "sysfs", "cgroup", "cgroup2", "devtmpfs") or source.startswith("/dev/") or \
            source in ("/", "/var/run/docker.sock") or any(fnmatch.fnmatch(target, w) for w in self.watch)
        if not risky:
            self.counts["events"] += 1
            return None
        sev = 0.9 if source.startswith("/dev/") or source == "/" else 0.7
        return self._raise("host_mount", sev, pid, comm, f"mount {source or fstype} on {target}")

    def detect_capability(self, pid: int, cap_effective: int, comm: str = ""):
        held = [c for c in DANGEROUS_CAPS if cap_effective >> CAP_BITS[c] & 1]
        if not held:
            self.counts["events"] += 1
            return None
        sev = 1.0 if "CAP_SYS_ADMIN" in held or "CAP_SYS_MODULE" in held else 0.6
        return self._raise("dangerous_capability", sev, pid, comm, ",".join(held))

    def check_file_access(self, path: str, pid: int = 0, comm: str = "", write: bool = False):
        for w in self.watch:
            if fnmatch.fnmatch(path, w):
                return self._raise("sensitive_file", 0.9 if write else 0.6, pid, comm, ("write " if write else "read ") + path)
        self.counts["events"] += 1
        return None

    def detect_syscall(self, pid: int, name: str, comm: str = ""):
        sev = DANGEROUS_SYSCALLS.get(name)
        if sev is None:
            self.counts["events"] += 1
            return None
        return self._raise("dangerous_syscall", sev, pid, comm, name)

    def add_watch_file(self, pattern: str) -> None:
        self.watch.append(pattern)

    def stats(self) -> dict:
        return dict(self.counts, alerts=len(self.alerts), max_severity=max((a.severity for a in self.alerts), default=0.0))

    def reset(self) -> None:
        self.alerts.clear()
        self.counts.clear()
        self.baseline_ns.clear()


class FunctionTableWatch:
    """Snapshot of a dispatch table; ``scan`` lists the names whose callable object was swapped or removed."""

    def __init__(self):
        self.tables: List[Tuple[dict, Dict[str, int]]] = []

    def watch(self, table: dict) -> int:
        self.tables.append((table, {k: id(v) for k, v in table.items()}))
        return len(self.tables) - 1

    def scan(self, index: Optional[int] = None) -> List[str]:
        out = []
        items = self.tables if index is None else [self.tables[index]]
        for table, snap in items:
            out += [k for k, i in snap.items() if k not in table or id(table[k]) != i]
            out += [k for k in table if k not in snap]
        return out

    def report(self) -> str:
        bad = self.scan()
        return "function tables intact" if not bad else "replaced or new entries: " + ", ".join(sorted(bad))


class AnomalyDetector:
    def __init__(self, alpha: float = 0.05, z_threshold: float = 4.0, warmup: int = 30):
        self.alpha, self.z, self.warmup = alpha, z_threshold, warmup
        self.state: Dict[str, List[float]] = {}      # metric -> [count, mean, variance]
        self.anomalies = 0

    def observe(self, metric: str, value: float) -> Optional[float]:
        """Feed one sample; returns its z-score when it is anomalous (and does not let it contaminate the baseline)."""
        st = self.state.setdefault(metric, [0, value, 0.0])
        n, mean, var = st
        if n >= self.warmup:
            z = (value - mean) / math.sqrt(max(var, 1e-12))
            if abs(z) > self.z:
                self.anomalies += 1
                return z
        a = self.alpha if n >= self.warmup else 1.0 / (n + 1)
        d = value - mean
        st[1] = mean + a * d
        st[2] = (1 - a) * (var + a * d * d)
        st[0] = n + 1
        return None

    def baseline(self, metric: str) -> Tuple[float, float]:
        _, m, v = self.state[metric]
        return m, math.sqrt(v)


class EventCorrelator:
    """``feed(detector, subject)`` from any monitor; an incident is raised when at least ``min_sources`` different
    detectors reported the same subject within ``window_s`` seconds."""

    def __init__(self, window_s: float = 60.0, min_sources: int = 2, clock: Callable[[], float] = time.time):
        self.window_s, self.min_sources, self.clock = window_s, min_sources, clock
        self.events: Dict[str, deque] = defaultdict(deque)
        self.incidents: List[dict] = []

    def feed(self, detector: str, subject: str, severity: float = 0.5) -> Optional[dict]:
        now = self.clock()
        q = self.events[subject]
        q.append((now, detector, severity))
        while q and q[0][0] < now - self.window_s:
            q.popleft()
        sources = {d for _, d, _ in q}
        if len(sources) >= self.min_sources:
            inc = {"subject": subject, "detectors": sorted(sources), "severity": min(1.0, max(s for _, _, s in q) + 0.1 * (len(sources) - 1)),
                   "time": now, "events": len(q)}
            self.incidents.append(inc)
            q.clear()
            return inc
        return None
