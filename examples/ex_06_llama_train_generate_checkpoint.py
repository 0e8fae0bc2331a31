"""A tiny Llama-shaped model end to end: a few training steps through ``TrainEngine`` (flat-buffer AdamW, fused
cross-entropy on CUDA), greedy generation, a ``.sneppx`` checkpoint written and read back."""
from _common import device, seed  # first: makes the package importable from a checkout
import os
import tempfile

import torch

from sneppx.checkpoint.sneppx_format import load_tensors, save_tensors, validate_checkpoint
from sneppx.models.config import ModelConfig
from sneppx.models.llama import LlamaForCausalLM
from sneppx.training.engine import TrainEngine


def main(steps: int = 40) -> dict:
    g, dev = seed(5), device()
    if dev.type == "cuda":      # the tensor-core kernels want head size 128 and widths that are multiples of 128
        cfg = ModelConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2,
                          num_key_value_heads=1, max_position_embeddings=64)
    else:
        cfg = ModelConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, max_position_embeddings=64)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = LlamaForCausalLM(cfg, dtype=dtype, device=dev)
    engine = TrainEngine(model, lr=3e-3, betas=(0.9, 0.95), weight_decay=0.0, max_grad_norm=1.0)
    # the task: continue an arithmetic progression modulo the vocabulary size
    start = torch.randint(0, 128, (32, 1), generator=g)
    stride = torch.randint(1, 4, (32, 1), generator=g)
    ids = ((start + stride * torch.arange(33)) % 128).to(dev)
    losses = [float(engine.step(ids[:, :-1], ids[:, 1:], shift_labels=False)) for _ in range(steps)]
    model.eval()
    prompt = ids[:2, :8]
    out = model.generate(prompt, max_new_tokens=6)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.sneppx")
        save_tensors(path, model.to_reference_state_dict(), metadata={"arch": "llama", "hidden_size": cfg.hidden_size})
        ok = validate_checkpoint(path)
        back, meta = load_tensors(path)
    same = all(torch.equal(back[k].cpu(), v.cpu()) for k, v in model.to_reference_state_dict().items())
    print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}; generated {out[0, 8:].tolist()} after {prompt[0].tolist()}; "
          f"checkpoint valid={ok}, {len(back)} tensors round-trip exactly={same}, metadata arch={meta['arch']}")
    return {"first": losses[0], "last": losses[-1], "valid": ok, "same": same}


if __name__ == "__main__":
    main()
