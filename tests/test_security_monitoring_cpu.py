"""S3 extensions: container-breakout rules, function-table watch, metric anomalies, event correlation."""
from sneppx_alg_b200.security.monitoring import (CAP_BITS, AnomalyDetector, BreakoutDetector, EventCorrelator,
                                                FunctionTableWatch)


class Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_breakout_rules():
    d = BreakoutDetector(clock=Clock())
    host = {"mnt": 4026531840, "pid": 4026531836, "net": 4026531992}
    cont = {"mnt": 4026532500, "pid": 4026532501, "net": 4026532502}
    d.record_namespaces(77, cont)
    assert d.detect_ns_change(77, cont, "python") is None
    a = d.detect_ns_change(77, dict(cont, mnt=host["mnt"]), "python", host_ns=host)
    assert a.kind == "namespace_change" and a.severity == 1.0 and "host" in a.detail
    assert d.detect_ns_change(77, dict(cont, mnt=host["mnt"], net=4026539999), "python", host_ns=host).severity == 0.6
    assert d.detect_mount(77, "/dev/sda1", "/mnt/x", "sh").severity == 0.9
    assert d.detect_mount(77, "", "/tmp/proc", "sh", fstype="proc").kind == "host_mount"
    assert d.detect_mount(77, "tmpfs", "/tmp/scratch", "sh", fstype="tmpfs") is None
    assert d.detect_capability(77, 1 << CAP_BITS["CAP_NET_RAW"], "ping") is None
    c = d.detect_capability(77, (1 << CAP_BITS["CAP_SYS_ADMIN"]) | (1 << CAP_BITS["CAP_SYS_PTRACE"]), "sh")
    assert c.severity == 1.0 and "CAP_SYS_ADMIN" in c.detail and "CAP_SYS_PTRACE" in c.detail
    assert d.check_file_access("/var/run/docker.sock", 77, "curl", write=True).severity == 0.9
    assert d.check_file_access("/sys/fs/cgroup/memory/release_agent", 77, "sh").kind == "sensitive_file"
    assert d.check_file_access("/home/user/data.bin", 77, "python") is None
    d.add_watch_file("/models/*.key")
    assert d.check_file_access("/models/prod.key") is not None
    assert d.detect_syscall(77, "finit_module", "insmod").severity == 0.9 and d.detect_syscall(77, "read", "cat") is None
    assert d.detect_syscall(1, "setns", "runc") is None                 # the runtime itself is allowed
    st = d.stats()
    assert st["alerts"] == 9 and st["allowed"] == 1 and st["max_severity"] == 1.0 and st["dangerous_syscall"] == 1
    d.reset()
    assert d.stats()["alerts"] == 0


def test_function_table_watch_and_anomalies_and_correlation():
    table = {"load": len, "save": print}
    w = FunctionTableWatch()
    i = w.watch(table)
    assert w.scan() == [] and w.report() == "function tables intact"
    table["save"] = lambda *a: None
    table["extra"] = sum
    del table["load"]
    assert sorted(w.scan(i)) == ["extra", "load", "save"] and "save" in w.report()
    ad = AnomalyDetector(alpha=0.1, z_threshold=4.0, warmup=20)
    vals = [100 + (i % 5) for i in range(60)]
    assert all(ad.observe("latency_ms", v) is None for v in vals)
    z = ad.observe("latency_ms", 400)
    assert z is not None and z > 4 and ad.anomalies == 1
    m, s = ad.baseline("latency_ms")
    assert 100 <= m <= 105 and s < 5                                     # the spike did not move the baseline
    assert ad.observe("latency_ms", 102) is None
    clock = Clock()
    ec = EventCorrelator(window_s=10, min_sources=2, clock=clock)
    assert ec.feed("breakout", "pid:77", 0.9) is None and ec.feed("breakout", "pid:77", 0.5) is None
    clock.t = 5
    inc = ec.feed("anomaly", "pid:77", 0.4)
    assert inc["detectors"] == ["anomaly", "breakout"] and inc["severity"] == 1.0 and inc["events"] == 3
    clock.t = 30
    assert ec.feed("tamper", "pid:77") is None                           # the earlier events were consumed / expired
