"""Drives the UNMODIFIED reference package (installed under ``baseline/_ref``) through its own public API and
reports, as one JSON object on stdout, what it can and cannot do towards the headline benchmark
(Llama-3-8B-shape bf16 ZeRO-3 training on GPUs). ``bench.py --impl reference`` runs this file in a child process
and puts the observations into its ``unavailable`` line; nothing here imports this repository's package.

Observed steps (each records ``ok`` or the exception text it raised):
  llama_forward      ``LlamaForCausalLM(config)`` of a scaled-down Llama-3 shape, ``forward(ids, labels=ids)``
  transformer_train  the generic ``Transformer``: forward, ``backward()``, ``AdamW.step()``; how many parameters got a
                     gradient and how many the optimizer changed; tokens/s of that loop on this CPU
  cuda_tensor        what ``Tensor.cuda()`` does (the array type that holds the data afterwards)
  collectives        ``init_process_group('nccl')`` + ``all_reduce``: world size seen and whether the result
                     differs from the input
"""
import json
import os
import sys
import time
import traceback


def _err():
    et, ev, tb = sys.exc_info()
    last = traceback.extract_tb(tb)[-1]
    return f"{et.__name__}: {ev} ({os.path.basename(last.filename)}:{last.lineno})"


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "_ref"))
    obs = {}
    try:
        import numpy as np
        import SneppX_ALG as sx
    except Exception:  # noqa: BLE001
        print(json.dumps({"import": _err()}))
        return 0
    obs["import"] = "ok"
    obs["version"] = getattr(sx, "__version__", None)
    rng = np.random.default_rng(0)
    # 1. the reference's Llama class on a scaled-down Llama-3 shape (GQA 4:2 heads, SwiGLU, theta 5e5)
    try:
        cfg = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, vocab_size=512, max_position_embeddings=64, head_dim=32, rope_theta=500000.0,
                   rms_norm_eps=1e-5)
        m = sx.LlamaForCausalLM(cfg)
        ids = sx.Tensor(rng.integers(0, 512, (1, 32)))
        out = m.forward(ids, labels=ids)
        out["loss"].backward()
        obs["llama_forward"] = "ok"
    except Exception:  # noqa: BLE001
        obs["llama_forward"] = _err()
    # 2. the generic Transformer: a whole training step, timed
    try:
        V, d, S, B = 1024, 128, 64, 2
        m = sx.Transformer(V, d, 4, 2, 4 * d, max_seq_len=S)
        params = list(m.parameters())
        opt = sx.AdamW(params, lr=1e-3)
        ids = sx.Tensor(rng.integers(0, V, (B, S)))

        def step():
            for p in params:
                p.grad = None
            loss = m(ids).sum()
            loss.backward()
            opt.step()

        before = [np.array(p.data).copy() for p in params]
        loss = m(ids).sum()
        loss.backward()
        with_grad = sum(getattr(p, "grad", None) is not None for p in params)
        opt.step()
        changed = sum(not np.array_equal(b, np.array(p.data)) for b, p in zip(before, params))
        t0 = time.perf_counter()
        n = 3
        for _ in range(n):
            step()
        dt = (time.perf_counter() - t0) / n
        obs["transformer_train"] = {"ok": True, "config": f"vocab {V}, d {d}, 4 heads, 2 layers, batch {B} x seq {S}, fp32 NumPy",
                                    "ms_per_step": dt * 1e3, "tokens_per_s": B * S / dt,
                                    "params": len(params), "params_with_grad_after_backward": with_grad,
                                    "params_changed_by_adamw_step": changed}
    except Exception:  # noqa: BLE001
        obs["transformer_train"] = _err()
    # 3. "CUDA" tensors
    try:
        t = sx.Tensor(np.arange(4, dtype=np.float32))
        c = t.cuda()
        data = getattr(c, "data", None)
        obs["cuda_tensor"] = {"device_attr": str(getattr(c, "device", None)),
                              "storage_type": type(data).__module__ + "." + type(data).__name__}
    except Exception:  # noqa: BLE001
        obs["cuda_tensor"] = _err()
    # 4. collectives
    try:
        sx.init_process_group("nccl")
        from SneppX_ALG.interface_bindings import distributed as rd
        t = sx.Tensor(np.arange(4, dtype=np.float32))
        r = sx.all_reduce(t)
        arr = r.numpy() if hasattr(r, "numpy") else np.asarray(getattr(r, "data", r))
        obs["collectives"] = {"world_size": int(rd.get_world_size()), "env_world_size": os.environ.get("WORLD_SIZE"),
                              "all_reduce_changed_values": bool(not np.array_equal(arr, np.arange(4, dtype=np.float32)))}
    except Exception:  # noqa: BLE001
        obs["collectives"] = _err()
    print(json.dumps(obs))
    return 0


if __name__ == "__main__":
    sys.exit(main())
