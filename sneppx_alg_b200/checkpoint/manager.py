"""Trainer-level checkpointing and the per-rank coordinated saver.

``CheckpointManager``: step / epoch / best metric / config / model / optimizer / RNG / scaler state, files
``checkpoint_{step}.ckpt|.sneppx`` and ``best_{step}_metric=...``, keep_last / keep_best pruning, ``load_latest`` /
``load_best`` (interface_bindings/checkpoint_manager.py:87-322). ``CheckpointCoordinator``: one file per rank
``checkpoint_{step}_rank_{rank}.sneppx`` with metadata {step, world_size, rank, ...}, barrier / save / barrier, background
writer, keep-last pruning (interface_bindings/checkpoint.py:208-316, kernel/distributed/checkpoint.c:241-376).
``reshard_flat``: re-slice ZeRO shards saved at one world size for another."""
from __future__ import annotations

import glob
import os
import pickle
import random
import re
from typing import Dict, List, Optional

import numpy as np
import torch

from .sneppx_format import AsyncSaver, load_tensors, save_tensors, validate_checkpoint


def _flatten_state(prefix, obj, tensors, meta):
    if torch.is_tensor(obj):
        tensors[prefix] = obj
        return {"__tensor__": prefix}
    if isinstance(obj, dict):
        return {str(k): _flatten_state(f"{prefix}.{k}", v, tensors, meta) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_flatten_state(f"{prefix}.{i}", v, tensors, meta) for i, v in enumerate(obj)]
    if isinstance(obj, (int, float, str, bool)) or obj is None:
        return obj
    return {"__pickle__": pickle.dumps(obj).hex()}


class UntrustedCheckpoint(RuntimeError):
    """The file holds a pickled Python object and the caller did not declare the file trusted."""


def _unflatten_state(node, tensors, trusted=False):
    if isinstance(node, dict):
        if "__tensor__" in node:
            return tensors[node["__tensor__"]]
        if "__pickle__" in node:
            if not trusted:
                raise UntrustedCheckpoint("checkpoint holds a pickled object; load it with trusted=True only if you "
                                          "wrote the file yourself (unpickling runs code from the file)")
            return pickle.loads(bytes.fromhex(node["__pickle__"]))
        return {k: _unflatten_state(v, tensors, trusted) for k, v in node.items()}
    if isinstance(node, list):
        return [_unflatten_state(v, tensors, trusted) for v in node]
    return node


class CheckpointManager:
    def __init__(self, directory: str, keep_last: int = 3, keep_best: int = 1, metric: str = "loss", mode: str = "min",
                 save_format: str = "binary", async_save: bool = False, rank: int = 0, world_size: int = 1,
                 barrier_fn=None, trusted: bool = False):
        """``world_size > 1`` makes the manager sharded: every rank writes its own
        ``checkpoint_{step}_rank_{rank}`` file between two barriers, a step counts as saved only when every rank's
        file exists and validates, and a loaded shard must carry the loading rank's number. ``trusted`` allows
        pickled nodes (arbitrary Python objects in the state) to be loaded; leave it off for files from elsewhere."""
        self.dir, self.keep_last, self.keep_best = directory, keep_last, keep_best
        self.metric, self.mode, self.format = metric, mode, save_format
        self.rank, self.world = rank, world_size
        self.barrier_fn = barrier_fn or (lambda: None)
        self.trusted = trusted or save_format != "binary"   # a pickle-format manager reads back its own pickles
        os.makedirs(directory, exist_ok=True)
        self.best: List[tuple] = []
        self.saver = AsyncSaver() if async_save and save_format == "binary" else None

    def _ext(self):
        return ".sneppx" if self.format == "binary" else ".ckpt"

    def _suffix(self, rank=None):
        return f"_rank_{self.rank if rank is None else rank}" if self.world > 1 else ""

    @staticmethod
    def _rng_state():
        """Generator states as plain data (ints, floats, tensors): nothing in it needs unpickling."""
        ver, keys, gauss = random.getstate()
        name, nkeys, pos, has_gauss, cached = np.random.get_state()
        st = {"python": {"version": int(ver), "keys": torch.tensor(list(keys), dtype=torch.int64), "gauss": gauss},
              "numpy": {"name": str(name), "keys": torch.from_numpy(np.asarray(nkeys, dtype=np.int64).copy()),
                        "pos": int(pos), "has_gauss": int(has_gauss), "cached": float(cached)},
              "torch": torch.get_rng_state()}
        if torch.cuda.is_available():
            st["cuda"] = list(torch.cuda.get_rng_state_all())
        return st

    @staticmethod
    def _set_rng_state(st):
        py, npst = st["python"], st["numpy"]
        if isinstance(py, dict):
            random.setstate((int(py["version"]), tuple(int(x) for x in py["keys"].tolist()), py["gauss"]))
            np.random.set_state((npst["name"], npst["keys"].numpy().astype(np.uint32), int(npst["pos"]),
                                 int(npst["has_gauss"]), float(npst["cached"])))
        else:   # tuple forms, as returned by random.getstate() / numpy.random.get_state()
            random.setstate(py)
            np.random.set_state(npst)
        torch.set_rng_state(st["torch"].cpu().to(torch.uint8))
        if "cuda" in st and torch.cuda.is_available():
            try:
                torch.cuda.set_rng_state_all([t.cpu().to(torch.uint8) for t in st["cuda"]])
            except (RuntimeError, IndexError):   # saved on a box with a different number of GPUs
                pass

    def save(self, step: int, model_state: dict, optimizer_state: Optional[dict] = None, epoch: int = 0,
             metrics: Optional[dict] = None, config: Optional[dict] = None, scaler_state: Optional[dict] = None,
             extra: Optional[dict] = None) -> str:
        state = {"step": step, "epoch": epoch, "best_metric": self.best[0][0] if self.best else None, "config": config,
                 "model_state": model_state, "optimizer_state": optimizer_state,
                 "rng": self._rng_state(),
                 "scaler_state": scaler_state, "metrics": metrics or {}, "extra": extra}
        state["shard_rank"], state["shard_world"] = self.rank, self.world
        path = os.path.join(self.dir, f"checkpoint_{step}{self._suffix()}{self._ext()}")
        self.barrier_fn()
        self._write(path, state)
        if self.world > 1:
            if self.saver:
                self.saver.wait()     # the closing barrier must mean "every rank's file is on disk"
            self.barrier_fn()
        if metrics and self.metric in metrics and self.keep_best > 0:
            val = float(metrics[self.metric])
            bpath = os.path.join(self.dir, f"best_{step}_{self.metric}={val:.6g}{self._suffix()}{self._ext()}")
            self._write(bpath, state)
            self.best.append((val, bpath))
            self.best.sort(key=lambda t: t[0], reverse=self.mode == "max")
            for _, p in self.best[self.keep_best:]:
                self._remove(p)
            self.best = self.best[: self.keep_best]
        self._prune()
        return path

    def _write(self, path, state):
        if self.format == "binary":
            tensors: Dict[str, torch.Tensor] = {}
            tree = _flatten_state("s", state, tensors, None)
            save_tensors(path, tensors, {"state_tree": tree, "format": "sneppx-trainer-1"}, saver=self.saver)
        else:
            with open(path + ".tmp", "wb") as f:
                pickle.dump(state, f)
            os.replace(path + ".tmp", path)

    def _remove(self, p):
        if self.saver:
            self.saver.wait()
        if os.path.exists(p):
            os.remove(p)

    def _prune(self):
        files = self.list_checkpoints()
        for _, p in files[: max(0, len(files) - self.keep_last)] if self.keep_last > 0 else []:
            self._remove(p)

    def list_checkpoints(self):
        """(step, this rank's path), oldest first; sharded: only steps for which every rank's file exists."""
        out = []
        for p in glob.glob(os.path.join(self.dir, "checkpoint_*")):
            if self.world > 1:
                m = re.search(rf"checkpoint_(\d+)_rank_{self.rank}\.(sneppx|ckpt)$", p)
                if m and all(os.path.exists(os.path.join(self.dir, f"checkpoint_{m.group(1)}_rank_{r}.{m.group(2)}"))
                             for r in range(self.world)):
                    out.append((int(m.group(1)), p))
                continue
            m = re.search(r"checkpoint_(\d+)\.(sneppx|ckpt)$", p)
            if m:
                out.append((int(m.group(1)), p))
        return sorted(out)

    def load(self, path: str, restore_rng: bool = True, trusted: Optional[bool] = None) -> dict:
        trusted = self.trusted if trusted is None else trusted
        if self.saver:
            self.saver.wait()
        if path.endswith(".sneppx"):
            tensors, meta = load_tensors(path)
            state = _unflatten_state(meta["state_tree"], tensors, trusted)
        else:
            if not trusted:
                raise UntrustedCheckpoint(".ckpt files are Python pickles; pass trusted=True for files you wrote")
            with open(path, "rb") as f:
                state = pickle.load(f)
        if self.world > 1 or state.get("shard_world", 1) not in (None, 1):
            if int(state.get("shard_world") or 1) != self.world:
                raise ValueError(f"checkpoint written by {state.get('shard_world')} ranks, loading with {self.world}")
            if int(state.get("shard_rank") or 0) != self.rank:
                raise ValueError(f"shard of rank {state.get('shard_rank')} loaded by rank {self.rank}")
        if restore_rng and state.get("rng"):
            rng = state["rng"]
            if isinstance(rng, str):      # older files carried the generator states as a pickle
                if not trusted:
                    raise UntrustedCheckpoint("generator state in this file is a pickle; pass trusted=True")
                rng = pickle.loads(bytes.fromhex(rng))
            self._set_rng_state(rng)
        return state

    def load_latest(self, **kw) -> Optional[dict]:
        files = self.list_checkpoints()
        for _, p in reversed(files):
            if not p.endswith(".sneppx") or validate_checkpoint(p):
                return self.load(p, **kw)
        return None

    def load_best(self, **kw) -> Optional[dict]:
        cands = glob.glob(os.path.join(self.dir, "best_*"))
        if not cands:
            return None

        def val(p):
            return float(re.search(r"=([-+0-9.eE]+?)\.(sneppx|ckpt)$", p).group(1))
        cands.sort(key=val, reverse=self.mode == "max")
        return self.load(cands[0], **kw)

    def close(self):
        if self.saver:
            self.saver.close()
            self.saver = None


class CheckpointCoordinator:
    """Per-rank sharded checkpoints with barriers before and after the save."""

    def __init__(self, directory: str, rank: int = 0, world_size: int = 1, keep_last: int = 2, async_save: bool = True,
                 barrier_fn=None):
        self.dir, self.rank, self.world, self.keep_last = directory, rank, world_size, keep_last
        os.makedirs(directory, exist_ok=True)
        self.saver = AsyncSaver() if async_save else None
        self.barrier_fn = barrier_fn or (lambda: None)

    def path(self, step: int, rank: Optional[int] = None) -> str:
        return os.path.join(self.dir, f"checkpoint_{step}_rank_{self.rank if rank is None else rank}.sneppx")

    def save(self, step: int, tensors: Dict[str, torch.Tensor], extra_meta: Optional[dict] = None) -> str:
        self.barrier_fn()
        meta = {"step": step, "world_size": self.world, "rank": self.rank}
        meta.update(extra_meta or {})
        p = self.path(step)
        save_tensors(p, tensors, meta, saver=self.saver)
        self.barrier_fn()
        self._prune()
        return p

    def wait(self):
        return self.saver.wait() if self.saver else 0

    def steps(self) -> List[int]:
        s = set()
        for p in glob.glob(os.path.join(self.dir, f"checkpoint_*_rank_{self.rank}.sneppx")):
            m = re.search(r"checkpoint_(\d+)_rank_", p)
            if m:
                s.add(int(m.group(1)))
        return sorted(s)

    def latest_complete_step(self) -> Optional[int]:
        """Newest step for which every rank's file exists and validates."""
        self.wait()
        for step in reversed(self.steps()):
            if all(os.path.exists(self.path(step, r)) and validate_checkpoint(self.path(step, r)) for r in range(self.world)):
                return step
        return None

    def load(self, step: int, rank: Optional[int] = None):
        self.wait()
        return load_tensors(self.path(step, rank))

    def _prune(self):
        if self.keep_last <= 0:
            return
        for s in self.steps()[: -self.keep_last]:
            self.wait()
            if os.path.exists(self.path(s)):
                os.remove(self.path(s))

    def close(self):
        if self.saver:
            self.saver.close()
            self.saver = None


def reshard_flat(shards: List[torch.Tensor], bounds: List[tuple], new_world: int) -> List[torch.Tensor]:
    """ZeRO shards of the bucketed flat layout (rank r holds slice r of every bucket, concatenated) saved with
    len(shards) ranks -> shards for ``new_world`` ranks."""
    old_world = len(shards)
    full_parts, off = [], 0
    for (b0, b1) in bounds:
        sz = (b1 - b0) // old_world
        full_parts.append(torch.cat([s[off: off + sz] for s in shards]))
        off += sz
    out = [[] for _ in range(new_world)]
    for part in full_parts:
        assert part.numel() % new_world == 0, "bucket size must divide by the new world size"
        sz = part.numel() // new_world
        for r in range(new_world):
            out[r].append(part[r * sz: (r + 1) * sz])
    return [torch.cat(x) for x in out]
