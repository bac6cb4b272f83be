"""Checkpoint audit: content hashes of everything a checkpoint holds, per section and per rank.

Two checkpoints that should be the same state (a run resumed half-way against the uninterrupted run; the same recipe
under two sharding strategies) are compared section by section instead of by loss curves
(reference: aspec/commands/_checkpoint_audit.py, tools/validation/dspark_cp_state_audit.py).  Sections: ``model``,
``optimizer.master``, ``optimizer.exp_avg``, ``optimizer.exp_avg_sq``, ``optimizer.step``, ``lr_scheduler``,
``rng.rank-N`` (torch, python, numpy and CUDA streams separately), ``work_state`` and the topology in ``meta``.
"""
from __future__ import annotations

import hashlib
import json
import os
import pickle
import warnings
from typing import Dict, Iterable, Tuple

import torch


def tensor_digest(named: Iterable[Tuple[str, torch.Tensor]]) -> dict:
    """sha256 over names, dtypes, shapes and bytes, in name order; ``coordinates`` counts the elements covered."""
    h = hashlib.sha256()
    count = 0
    for name, t in sorted(named, key=lambda kv: kv[0]):
        t = t.detach().cpu().contiguous()
        h.update(f"{name}|{t.dtype}|{tuple(t.shape)}|".encode())
        h.update(t.reshape(-1).view(torch.uint8).numpy().tobytes())
        count += t.numel()
    return {"sha256": h.hexdigest(), "coordinates": count}


def _load_dcp(path: str) -> dict:
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict_from_keys
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        return _load_state_dict_from_keys(checkpoint_id=path)


def _blob_digest(obj) -> str:
    if torch.is_tensor(obj):
        return tensor_digest([("t", obj)])["sha256"]
    return hashlib.sha256(pickle.dumps(obj, protocol=4)).hexdigest()


def checkpoint_hashes(ckpt_dir: str) -> Dict[str, dict]:
    if not os.path.isfile(os.path.join(ckpt_dir, "complete.json")):
        raise FileNotFoundError(f"{ckpt_dir} is not a published checkpoint (no complete.json)")
    out: Dict[str, dict] = {}
    model = _load_dcp(os.path.join(ckpt_dir, "model"))["model_state"]
    out["model"] = tensor_digest(model.items())
    optim = _load_dcp(os.path.join(ckpt_dir, "optimizer"))["optim_state"]
    for group in ("master", "exp_avg", "exp_avg_sq"):
        out[f"optimizer.{group}"] = tensor_digest((k.split(".", 1)[1], v) for k, v in optim.items() if k.startswith(group + "."))
    out["optimizer.step"] = {"value": int(optim["step"])}
    sched = _load_dcp(os.path.join(ckpt_dir, "lr_scheduler"))["lr_scheduler"]
    out["lr_scheduler"] = {"last_epoch": int(sched["last_epoch"])}
    rng_dir = os.path.join(ckpt_dir, "rng")
    for name in sorted(os.listdir(rng_dir)):
        state = torch.load(os.path.join(rng_dir, name), weights_only=False)
        out[f"rng.{name[:-3]}"] = {k: _blob_digest(v) for k, v in state.items() if k in ("torch", "cuda", "numpy", "python")} | \
            {"rank": state.get("rank"), "world_size": state.get("world_size")}
    work = json.load(open(os.path.join(ckpt_dir, "work_state.json")))
    out["work_state"] = {"sha256": hashlib.sha256(json.dumps(work, sort_keys=True).encode()).hexdigest(),
                         "optimizer_step": work.get("optimizer_step")}
    meta = json.load(open(os.path.join(ckpt_dir, "meta.json")))
    out["meta"] = {"iteration": meta.get("iteration"), "world_size": meta.get("world_size"),
                   "topology_sha256": hashlib.sha256(json.dumps(meta.get("training_topology"), sort_keys=True).encode()).hexdigest()}
    return out


def compare(a: Dict[str, dict], b: Dict[str, dict], ignore: Iterable[str] = ()) -> Dict[str, tuple]:
    """Sections that differ (``{section: (a, b)}``); sections whose name starts with an ``ignore`` prefix are skipped."""
    skip = tuple(ignore)
    diff = {}
    for key in sorted(set(a) | set(b)):
        if skip and key.startswith(skip):
            continue
        if a.get(key) != b.get(key):
            diff[key] = (a.get(key), b.get(key))
    return diff
