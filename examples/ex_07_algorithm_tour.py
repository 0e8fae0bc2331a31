"""The five algorithm families on small shapes: HSS state-space scan, SER sparse expert routing, ARC input guard /
output verifier with an FGSM probe, an NPE program compiled and run on the register VM, FM federated memory sync; then
the composed pipeline model trained for a few steps on its regression objective."""
from _common import device, seed  # first: makes the package importable from a checkout
import torch

import SneppX_ALG as sx
from sneppx.algorithms import npe
from sneppx.algorithms.arc import ARCLayer, simulate_attack
from sneppx.algorithms.fm import FMController
from sneppx.algorithms.hss import HSSModel
from sneppx.algorithms.pipeline import Model, ModelConfig
from sneppx.algorithms.ser import SERLayer


def main() -> dict:
    seed(6)
    dev = device()
    out = {}
    x = torch.randn(2, 32, 64, device=dev)
    hss = HSSModel(state_dim=16, input_dim=64, output_dim=64, num_layers=2, seq_len=32, device=dev)
    out["hss"] = tuple(hss(x).shape)
    ser = SERLayer(num_experts=4, top_k=2, input_dim=64, hidden_dim=128, output_dim=64, device=dev)
    y = ser(x)
    out["ser"] = (tuple(y.shape), round(ser.aux_loss.item(), 4))
    arc = ARCLayer(64, device=dev)
    clean = arc(x)
    loss_fn = lambda v: arc(v).float().pow(2).mean()          # noqa: E731
    adv = simulate_attack(x, epsilon=0.05, loss_fn=loss_fn, lo=-10.0, hi=10.0)
    with torch.no_grad():
        shift = (arc(adv) - clean).abs().mean().item()
    out["arc"] = {"metrics": [round(m, 3) for m in arc.metrics.tolist()], "fgsm_shift": round(shift, 4)}
    w = {"w1": torch.randn(64, 32) / 8, "b1": torch.zeros(32), "w2": torch.randn(32, 64) / 6}
    prog = sx.NPECompiler().compile([{"type": "matmul", "args": ["x", "w1"], "dest": "h"}, {"type": "add", "args": ["h", "b1"], "dest": "h2"},
                                     {"type": "relu", "args": ["h2"], "dest": "a"}, {"type": "matmul", "args": ["a", "w2"], "dest": "y"}], w)
    fused = sx.NPECompiler().jit_optimize(prog)
    vm = npe.VM()
    vm.load(fused)
    xin = torch.randn(4, 64)
    out["npe"] = {"instructions": (len(prog.instructions), len(fused.instructions)),
                  "matches_torch": bool(torch.allclose(vm.run(xin), torch.relu(xin @ w["w1"]) @ w["w2"], atol=1e-4))}
    fm = FMController(num_nodes=3, memory_dim=64, memory_capacity=32, sync_interval=0, device=dev)
    for node in range(3):
        fm(torch.randn(1, 64, device=dev) + node, node_id=node)
    out["fm_sync_status"] = fm.sync()
    model = Model(ModelConfig(input_dim=64, output_dim=64, vocab_size=50, num_heads=4, enable_ser=True,
                              hss=hss.cfg.__class__(state_dim=16, num_layers=1, seq_len=16),
                              ser=ser.cfg.__class__(num_experts=4, top_k=2, hidden_dim=128)), device=dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    ids = torch.randint(0, 50, (4, 16), device=dev)
    target = torch.randn(4, 16, 64, device=dev)
    losses = []
    for _ in range(25):
        opt.zero_grad()
        loss = model.train_step_loss(ids, target)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    out["pipeline_loss"] = (round(losses[0], 3), round(losses[-1], 3))
    for k, v in out.items():
        print(f"{k}: {v}")
    return out


if __name__ == "__main__":
    main()
