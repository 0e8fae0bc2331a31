"""HSS / SER / ARC / NPE / FM and the unified pipeline on CPU (shape, equality of scan variants, oracle checks),
following the reference's unit and integration tests (tests/unit/hss/test_hss_parallel_scan.c,
tests/integration/test_hss_ser_arc_stack.c, test_full_pipeline.c)."""
import torch

from sneppx_alg_b200 import algorithms as A


def test_hss_scan_variants_agree_and_discretise():
    torch.manual_seed(0)
    s, i, o, L = 8, 6, 5, 37
    Am = -torch.diag(torch.rand(s) + 0.5) + 0.05 * torch.randn(s, s)
    B, C, D, dt = torch.randn(s, i), torch.randn(o, s), torch.randn(o, i), torch.rand(s) * 0.1 + 0.01
    Ab, Bb = A.HSSDiscretize.euler(Am, B, dt)
    assert torch.allclose(Ab, torch.eye(s) + dt[:, None] * Am) and torch.allclose(Bb, dt[:, None] * B)
    Az, _ = A.HSSDiscretize.zoh(Am, B, dt)
    assert torch.allclose(Az, Ab, atol=2e-2)                       # first-order agreement
    At, _ = A.HSSDiscretize.bilinear(Am, B, dt)
    assert torch.allclose(At, Az, atol=1e-3)
    x = torch.randn(3, L, i)
    y_seq, h_seq = A.HSSScan.sequential(Ab, Bb, C, D, x)
    y_par, h_par = A.HSSScan.parallel_scan(Ab, Bb, C, D, x)
    assert torch.allclose(y_seq, y_par, atol=1e-4) and torch.allclose(h_seq, h_par, atol=1e-4)
    # step-by-step decode matches the scan
    h = torch.zeros(3, s)
    for t in range(L):
        y_t, h = A.HSSStep.step(h, x[:, t], Ab, Bb, C, D)
    assert torch.allclose(y_t, y_seq[:, -1], atol=1e-4)
    # carried state: scanning two halves equals scanning the whole
    y1, h1 = A.HSSScan.parallel_scan(Ab, Bb, C, D, x[:, :20])
    y2, _ = A.HSSScan.parallel_scan(Ab, Bb, C, D, x[:, 20:], h0=h1)
    assert torch.allclose(torch.cat([y1, y2], 1), y_seq, atol=1e-4)


def test_hss_model_trains():
    torch.manual_seed(0)
    m = A.HSSModel(A.HSSConfig(state_dim=8, input_dim=16, output_dim=16, num_layers=2))
    assert m.num_params_per_layer() == 9
    x = torch.randn(2, 12, 16)
    opt = torch.optim.Adam(m.parameters(), 1e-2)
    losses = []
    for _ in range(30):
        loss = (m(x) - x.flip(-1)).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < 0.7 * losses[0]


def test_ser_routing_and_layer():
    torch.manual_seed(0)
    logits = torch.randn(64, 8)
    idx, w, probs, counts = A.SERRoute.topk_gating(logits, 2)
    assert idx.shape == (64, 2) and torch.allclose(w.sum(-1), torch.ones(64), atol=1e-5) and int(counts.sum()) == 128
    ref = torch.topk(torch.softmax(logits, -1), 2).indices
    assert torch.equal(idx.long().sort(-1).values, ref.sort(-1).values)
    lb = A.SERRoute.load_balance_loss(probs, counts, 2)
    assert float(lb) >= 0.99                                        # equals 1 for a perfectly uniform router
    assert torch.allclose(A.SERLoss.z_loss(logits), logits.pow(2).mean())
    for act in ("relu", "swiglu"):
        layer = A.SERLayer(A.SERConfig(num_experts=4, top_k=2, input_dim=16, hidden_dim=32, output_dim=16, activation=act))
        y = layer(torch.randn(2, 5, 16))
        assert y.shape == (2, 5, 16) and torch.isfinite(y).all() and torch.isfinite(layer.aux_loss)
        (y.sum() + layer.aux_loss).backward()


def test_arc():
    torch.manual_seed(0)
    layer = A.ARCLayer(16)
    x = torch.randn(8, 16)
    y = layer(x)
    assert y.shape == x.shape and layer.metrics.shape == (4,) and torch.isfinite(layer.metrics).all()
    w = torch.randn(16)
    adv = A.simulate_attack(x.clamp(-1, 1), 1, 0.1, loss_fn=lambda z: (z @ w).sum())
    assert torch.allclose(adv, (x.clamp(-1, 1) + 0.1 * w.sign()).clamp(-1, 1))      # FGSM = x + eps * sign(grad)
    pgd = A.simulate_attack(x.clamp(-1, 1), 2, 0.1, loss_fn=lambda z: (z @ w).sum())
    assert float((pgd - x.clamp(-1, 1)).abs().max()) <= 0.1 + 1e-6
    ob = A.GradientObfuscator(noise_scale=0.0, clip_max=0.5)
    g = ob(torch.tensor([2.0, -3.0, 0.1]))
    assert torch.allclose(g, torch.tensor([0.5, -0.5, 0.1])) and abs(ob.clamp_ratio - 2 / 3) < 1e-6


def test_npe_vm_compiler_verifier_jit():
    torch.manual_seed(0)
    prog = A.compile_mlp(8, 16)
    ok, msgs = A.verify_program(prog)
    assert ok and not msgs
    vm = A.NPEVM()
    vm.load(prog)
    x = torch.randn(5, 8)
    y = vm.run(x)
    mem = prog.memory
    W1, b1 = mem[:128].view(8, 16), mem[128:144]
    W2, b2 = mem[144:272].view(16, 8), mem[272:280]
    ref = torch.relu(x @ W1 + b1) @ W2 + b2
    assert torch.allclose(y, ref, atol=1e-5)
    n0 = len(vm.program.instructions)
    opt = vm.optimize()
    assert len(opt.instructions) < n0 and any(i.opcode == A.Op.FUSED_LINEAR for i in opt.instructions)
    assert torch.allclose(vm.run(x), ref, atol=1e-5)
    bad = A.NPEProgram(4)
    bad.append(A.Instruction(A.Op.LOAD, 17, immediate=99)).append(A.Instruction(A.Op.BRANCH, immediate=7))
    ok, msgs = A.verify_program(bad)
    assert not ok and len(msgs) >= 3
    att = A.NPELayer(8, kind="attention", seq_len=6)
    assert att(torch.randn(6, 8)).shape == (6, 8)
    layer = A.NPELayer(8, 16)
    layer(x).sum().backward()
    assert layer.program.memory.grad is not None and layer.program.memory.grad.abs().sum() > 0


def test_fm():
    torch.manual_seed(0)
    c = A.FMController(A.FMConfig(num_nodes=3, memory_dim=8, memory_capacity=4, sync_interval=0))
    k = torch.randn(8)
    bank = c.nodes[0].bank
    bank.write(k, k * 2)
    assert torch.allclose(bank.read(k), k * 2) and bank.read(k + 10) is None
    for j in range(6):                                   # beyond capacity -> eviction keeps size bounded
        bank.write(torch.randn(8) * 5 + 20 * j, torch.ones(8) * j)
    assert bank.num_entries == 4
    for n in c.nodes:
        n.bank.write(torch.zeros(8), torch.full((8,), float(n.node_id)))
    v0 = torch.stack([n.bank.values[0] for n in c.nodes])
    c.sync_all_reduce()
    assert all(torch.allclose(n.bank.values[0], v0.mean(0)) for n in c.nodes)
    g = torch.tensor([0.1, -5.0, 0.2, 3.0, 0.0, 0.05, -0.3, 1.0])
    assert (A.compress_topk(g, 0.25) != 0).sum() == 2
    ef = c.error_feedback[0]
    ef.ratio = 0.25
    s = ef.compress(g)
    assert torch.allclose(s + ef.residual, g)
    assert 10 <= c.adaptive_sync_interval(100.0) <= 200
    x = torch.randn(1, 8)
    y1 = c(x, 1)
    y2 = c(x, 1)                                        # second call blends with the stored memory
    assert torch.allclose(y1, x) and torch.allclose(y2, x, atol=1e-5)
    c.sync_gossip(2, seed=0)
    c.sync_topology()


def test_full_pipeline_shapes_and_gradients():
    torch.manual_seed(0)
    cfg = A.ModelConfig(input_dim=32, output_dim=32, vocab_size=50, num_heads=4, enable_ser=True, enable_arc=True,
                        enable_npe=True, enable_fm=True,
                        hss=A.HSSConfig(state_dim=8, num_layers=1),
                        ser=A.SERConfig(num_experts=4, hidden_dim=64), fm=A.FMConfig(num_nodes=2, memory_capacity=8))
    m = A.Model(cfg)
    ids = torch.randint(0, 50, (2, 10))
    y = m(ids)
    assert y.shape == (2, 10, 32) and torch.isfinite(y).all()
    loss = m.train_step_loss(ids, torch.zeros(2, 10, 32))
    loss.backward()
    assert m.embed.weight.grad is not None and m.hss.layers[0].A.grad is not None
    d = A.Model()                                      # defaults: attention + HSS only
    assert d.ser is None and d.arc is None and d.npe is None and d.fm is None and d.hss is not None
