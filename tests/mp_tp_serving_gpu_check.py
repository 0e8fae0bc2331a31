"""Worker for the 2-GPU tensor-parallel serving test (run under torch.distributed.run): the TP engine (peer-load
all-reduce kernel, CUDA-graph decode) against the single-GPU engine on the same bf16 model: first-token logits agree
within bf16 reduction noise, and wherever a greedy continuation leaves the single-GPU one the two candidate tokens are a
near tie in the single-GPU engine's own logits for that prefix (a different summation order can flip an argmax
between two nearly equal logits; everything after such a flip differs legitimately)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from sneppx_alg_b200.models import ModelConfig, build_model  # noqa: E402
from sneppx_alg_b200.ops import check_status  # noqa: E402
from sneppx_alg_b200.serving.llm_engine import LLMEngine, SamplingParams, TPLlamaPagedRunner  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=512, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=4,
                      intermediate_size=1024, vocab_size=2048, max_position_embeddings=512, rms_norm_eps=1e-5)
    model = build_model(cfg, dtype=torch.bfloat16, device=dev).eval()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (40, 7, 130, 64, 19)]
    sp = SamplingParams(max_new_tokens=24)
    ref = LLMEngine(model, num_blocks=256, block_size=16, max_batch_size=4, max_model_len=512)
    want = ref.generate(prompts, sp)
    eng = LLMEngine(model, num_blocks=256, block_size=16, max_batch_size=4, tp_group=dist.group.WORLD, max_model_len=512)
    assert isinstance(eng.runner, TPLlamaPagedRunner) and eng.runner._sg is not None
    got = eng.generate(prompts, sp)
    graphs = len(getattr(eng.runner, "_graphs", None) or {})
    # logits of the first generated position, both engines, same prompt
    ref.cache.add_sequence(10_000, None)
    eng.cache.add_sequence(10_000, None)
    l_ref = ref.runner.prefill(10_000, prompts[2], 0)
    l_tp = eng.runner.prefill(10_000, prompts[2], 0)
    rel = (l_ref - l_tp).abs().max().item() / (l_ref.abs().max().item() + 1e-6)
    agree = sum(a == b for w, o in zip(want, got) for a, b in zip(w, o)) / sum(len(w) for w in want)
    # first divergence of every sequence: the single-GPU logits for that prefix must hold the two tokens within noise
    ties_ok, sid = True, 20_000
    for pr, w, o in zip(prompts, want, got):
        i = next((j for j, (a, b) in enumerate(zip(w, o)) if a != b), None)
        if i is None:
            continue
        sid += 1
        ref.cache.add_sequence(sid, None)
        lg = ref.runner.prefill(sid, pr + w[:i], 0)[0]
        ref.cache.free_sequence(sid)
        gap = (lg[w[i]] - lg[o[i]]).abs().item() / (lg.abs().max().item() + 1e-6)
        ties_ok = ties_ok and gap < 3e-2
    torch.cuda.synchronize()
    check_status()
    ok = rel < 3e-2 and ties_ok and agree >= 0.3 and graphs >= 1 and all(len(o) == 24 for o in got)
    t = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    same = torch.tensor([hash(tuple(map(tuple, got))) % (1 << 30)], device=dev)
    lo, hi = same.clone(), same.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ranks_agree = bool(lo.item() == hi.item())           # every rank must sample the same tokens
    if rank == 0:
        print(f"tp serving world {world}: logits rel err {rel:.3e}, token agreement with 1 GPU {agree:.3f} (divergences are near ties: {ties_ok}), decode graphs {graphs}, "
              f"ranks agree {ranks_agree} ->", "OK" if (t.item() and ranks_agree) else "MISMATCH", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if (t.item() and ranks_agree) else 1)


if __name__ == "__main__":
    try:
        main()
    except SystemExit:
        raise
    except BaseException:  # noqa: BLE001  (the launcher only keeps the tail of stderr: put the cause on stdout)
        import traceback
        print("WORKER ERROR on rank", os.environ.get("RANK"), flush=True)
        traceback.print_exc(file=sys.stdout)
        sys.stdout.flush()
        os._exit(1)
