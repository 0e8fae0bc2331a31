"""C++ host runtime: TCP ring all-reduce / param sync across processes, heartbeat failure detection with a host-side
injected failure (a rank stops announcing itself), elastic membership rules, checkpoint container."""
import os
import time

import numpy as np
import torch
import torch.multiprocessing as mp

from sneppx_alg_b200.checkpoint.sneppx_format import (AsyncSaver, CheckpointReader, CheckpointWriter, load_tensors,
                                                      save_tensors, validate_checkpoint)
from sneppx_alg_b200.parallel.host_runtime import (ALIVE, DEAD, ElasticMembership, ElasticTrainer,
                                                   FaultToleranceManager, HeartbeatMonitor, TcpRing)


def _ring_worker(rank, world, base, q):
    addrs = [f"127.0.0.1:{base + r}" for r in range(world)]
    ring = TcpRing(rank, world, addrs)
    x = np.arange(1000, dtype=np.float32) * (rank + 1)
    ring.all_reduce(x)
    s = np.full(7, float(rank), dtype=np.float32)
    ring.all_reduce(s, average=False)
    p = np.full(5, float(rank), dtype=np.float32)
    ver = ring.sync_params(p, version=10 + (1 if rank == 1 else 0))
    q.put((rank, float(x[10]), float(s[0]), p.tolist(), ver))
    ring.shutdown()


def test_tcp_ring_all_reduce_and_param_sync():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    base = 31000 + os.getpid() % 2000
    world = 3
    procs = [ctx.Process(target=_ring_worker, args=(r, world, base, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    for rank, x10, s0, pvals, ver in res:
        assert abs(x10 - 10 * (1 + 2 + 3) / 3) < 1e-4          # average
        assert s0 == 0 + 1 + 2                                  # sum
        assert pvals == [1.0] * 5 and ver == 11                 # highest version (rank 1) wins everywhere


def _hb_worker(rank, base, q, fail_after):
    hb = HeartbeatMonitor(rank, 2, base_port=base, interval_s=0.05, timeout_s=0.25).start()
    t0 = time.time()
    seen = []
    while time.time() - t0 < 2.5:
        if rank == 1 and time.time() - t0 > fail_after:
            hb.pause_sending(True)          # injected failure: rank 1 goes silent
        seen.append(hb.status(1 - rank))
        time.sleep(0.05)
    q.put((rank, seen))
    if rank == 0:
        time.sleep(2.0)                     # keep announcing while the other process, which may have started later, samples
    hb.stop()


def test_heartbeat_detects_silent_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    base = 33000 + os.getpid() % 2000
    procs = [ctx.Process(target=_hb_worker, args=(r, base, q, 0.8)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=30) for _ in range(2))
    for p in procs:
        p.join(10)
    assert ALIVE in res[0] and res[0][-1] == DEAD               # rank 0 saw rank 1 alive, then dead
    assert res[1][-1] == ALIVE                                  # rank 0 kept announcing itself


def test_elastic_membership_and_recovery():
    m = ElasticMembership(4, self_rank=0)
    assert not m.leave(0)                                       # cannot remove itself
    restored = []
    tr = ElasticTrainer(m, restore_fn=lambda v: restored.append(v) or True)
    tr.mark_checkpoint(7)
    assert tr.handle_failure([2])
    assert m.members == [0, 1, 3] and m.new_topology() == {0: 0, 1: 1, 3: 2} and restored == [6]
    assert tr.handle_failure([3])
    assert not m.leave(1)                                       # would drop below half of the original world
    assert m.join(5) and m.members == [0, 1, 5]

    class FakeMonitor:
        def dead_ranks(self):
            return [1]
    ft = FaultToleranceManager(FakeMonitor(), ElasticTrainer(ElasticMembership(4, 0), lambda v: True))
    assert ft.poll() == {0: 0, 2: 1, 3: 2} and ft.poll() is None


def test_checkpoint_container_roundtrip_and_corruption(tmp_path):
    path = str(tmp_path / "c.sneppx")
    tensors = {"w": torch.randn(4, 6), "b16": torch.randn(3, 5).bfloat16(), "idx": torch.arange(7), "s": torch.tensor(3.5)}
    save_tensors(path, tensors, {"step": 12, "world_size": 1})
    assert validate_checkpoint(path)
    back, meta = load_tensors(path)
    assert meta["step"] == 12 and list(back) == list(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and torch.equal(back[k], tensors[k])
    raw = bytearray(open(path, "rb").read())
    raw[0] ^= 0xFF
    bad = str(tmp_path / "bad.sneppx")
    open(bad, "wb").write(raw)
    assert not validate_checkpoint(bad)
    open(bad, "wb").write(open(path, "rb").read()[:-5])          # truncated file
    assert not validate_checkpoint(bad)
    saver = AsyncSaver(max_pending=2)
    for i in range(4):
        save_tensors(str(tmp_path / f"a{i}.sneppx"), {"x": torch.full((1000,), float(i))}, {"i": i}, saver=saver)
    assert saver.wait() == 0
    saver.close()
    assert load_tensors(str(tmp_path / "a3.sneppx"))[0]["x"][0] == 3.0
    w = CheckpointWriter(str(tmp_path / "raw.sneppx"))
    w.write_tensor(np.arange(6, dtype=np.float32).tobytes(), (2, 3), 0)
    w.close()
    r = CheckpointReader(str(tmp_path / "raw.sneppx"))
    assert r.tensor_info(0) == ((2, 3), 0, 24) and r.read_metadata() == {}
    r.close()
