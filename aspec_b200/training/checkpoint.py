"""Two-phase checkpoints with exact-resume identity.

Layout (reference: aspec/training/checkpoint.py:260-300, 546-651, 1066-1132)::

    <output_dir>/checkpoints/
      .iter_0000009.incomplete/          staging while ranks write
      iter_0000009/
        model/         torch.distributed.checkpoint, key "model_state"
        optimizer/     DCP "optim_state": AdamW moments + fp32 masters by parameter name
        lr_scheduler/  DCP
        rng/rank-00000.pt ...   {schema aspec.rng-state/v1, torch, cuda, numpy?, python}
        meta.json  draft_config.json  work_state.json  complete.json
      latest_checkpointed_iteration.txt

``save`` stages the shards; after the optimizer step has been committed the driver calls ``publish``,
which writes ``work_state.json``, verifies every required file (all RNG ranks included), writes
``complete.json`` and renames staging -> final atomically.  ``load`` refuses a checkpoint without
``complete.json`` and, for exact resume, any change of logical topology / objective / model semantics;
``continual_training`` loads weights only and re-derives the fp32 masters.

The directory layout and the two-phase protocol are the reference's; the file contents are this framework's own (schema
tags under ``schema``, the optimizer as flat ``master / exp_avg / exp_avg_sq`` maps by parameter name, the scheduler as
one ``last_epoch``).  Training checkpoints are therefore not interchangeable with the reference's in either direction;
what is interchangeable are the exports (``commands/convert_to_hf.py``: HF and serving layouts with the reference's
tensor names) and weights-only starts from such an export.
"""
from __future__ import annotations

import json
import os
import random
import shutil
import time
import warnings
from typing import Any, Mapping, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from aspec_b200.config.draft_config import draft_model_semantics, resolve_draft_algorithm
from aspec_b200.config.draft_attention import resolve_attention_policy
from aspec_b200.config.draft_structure import resolve_ffn_policy

RNG_SCHEMA = "aspec.rng-state/v1"
WORK_SCHEMA = "aspec.checkpoint-work-state/v1"
COMPLETE_SCHEMA = "aspec.checkpoint-completion/v1"
TRACKER = "latest_checkpointed_iteration.txt"
# execution bounds that may change between save and resume
_IGNORED_OBJECTIVE_KEYS = ("dsa_workspace_bytes", "csa_workspace_bytes", "qsa_workspace_bytes", "loss_chunk_size")


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def iteration_dir(output_dir: str, step_id: int, staging: bool = False) -> str:
    name = f"iter_{int(step_id):07d}"
    return os.path.join(output_dir, "checkpoints", f".{name}.incomplete" if staging else name)


def training_objective(args: Mapping[str, Any], algorithm: str) -> dict:
    g = args.get
    common = {k: g(k) for k in ("max_seq_length", "micro_batch_size", "draft_accumulation_steps",
                                "max_grad_norm", "seed") if g(k) is not None}
    if algorithm in ("dflash", "dspark", "dflash2"):
        keys = ["block_size", "anchor_sampling_scope", "num_anchors", "num_target_layers", "loss_decay_gamma",
                "ce_loss_alpha", "l1_loss_alpha", "deterministic_anchor_sampling"]
        if algorithm == "dspark":
            keys += ["confidence_head_alpha", "l1_target_temperature", "l1_target_top_p", "l1_target_top_k",
                     "l1_draft_temperature", "l1_draft_top_p", "l1_draft_top_k"]
    elif algorithm in ("eagle3", "eagle4"):
        keys = ["ttt_length", "loss_type", "lk_eta", "ploss_weights", "freeze_lm_head"]
    else:
        keys = ["mtp_steps", "step_weight_beta", "step_weights"]
    return {**common, **{k: g(k) for k in keys if g(k) is not None}}


def logical_training_topology(args: Mapping[str, Any], draft_config) -> dict:
    raw = draft_config.to_dict() if hasattr(draft_config, "to_dict") else dict(draft_config)
    algorithm = resolve_draft_algorithm(raw)
    policy = resolve_attention_policy(raw) if algorithm not in ("mtp",) else {}
    g = args.get
    return {
        "world_size": int(g("world_size", _world())),
        "training_num_nodes": int(g("training_num_nodes", 1)),
        "training_num_gpus_per_node": int(g("training_num_gpus_per_node", g("world_size", _world()))),
        "attention_backend": g("attention_backend", "sm100_flash"),
        "draft_context_parallel_size": int(g("draft_context_parallel_size", 1)),
        "sp_ulysses_size": int(g("sp_ulysses_size", 1)), "sp_ring_size": int(g("sp_ring_size", 1)),
        "fsdp_strategy": g("fsdp_strategy", "REPLICATE"),
        "draft_algorithm": algorithm,
        "training_objective": training_objective(args, algorithm),
        "draft_attention_windows": policy.get("context_windows"),
        "draft_attention_policy": {k: policy.get(k) for k in ("layer_types", "window_semantics", "draft_block_attention",
                                                                "csa", "qsa", "dsa") if policy.get(k) is not None},
        "draft_model_semantics": draft_model_semantics(raw),
        "draft_ffn_policy": resolve_ffn_policy(raw) if algorithm != "mtp" else {"ffn_type": "dense"},
    }


def _strip_bounds(value):
    if isinstance(value, dict):
        return {k: _strip_bounds(v) for k, v in value.items() if k not in _IGNORED_OBJECTIVE_KEYS
                and k != "workspace_bytes"}
    return value


def validate_exact_resume_topology(saved: Mapping[str, Any], current: Mapping[str, Any]) -> None:
    """Every field the checkpoint recorded must equal the current one (objective: sub-dict containment)."""
    problems = []
    for key, old in saved.items():
        new = current.get(key)
        if key == "training_objective":
            for k, v in _strip_bounds(old).items():
                if _strip_bounds(new or {}).get(k) != v:
                    problems.append(f"training_objective.{k}: checkpoint={v!r} current={(new or {}).get(k)!r}")
        elif _strip_bounds(old) != _strip_bounds(new):
            problems.append(f"{key}: checkpoint={old!r} current={new!r}")
    if problems:
        raise ValueError("Exact resume refused: the run differs from the checkpoint in\n  " + "\n  ".join(problems)
                         + "\nUse training.continual_training=true for a weights-only new phase.")


def _rng_state() -> dict:
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    state = {"schema": RNG_SCHEMA, "rank": _rank(), "world_size": world,
             "torch": torch.get_rng_state(), "python": random.getstate()}
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state()
    try:
        import numpy as np
        state["numpy"] = np.random.get_state()
    except Exception:  # pragma: no cover
        pass
    return state


def _restore_rng(state: dict) -> None:
    if state.get("schema") != RNG_SCHEMA:
        raise ValueError("unknown RNG state schema")
    # a generator stream belongs to one rank of one world size: a file moved between ranks would replay another
    # rank's anchors (files written before the two fields existed carry neither and are taken as they are)
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if "rank" in state and (state["rank"] != _rank() or state.get("world_size") != world):
        raise ValueError(f"RNG state of rank {state['rank']} / world {state.get('world_size')} offered to "
                         f"rank {_rank()} / world {world}")
    torch.set_rng_state(state["torch"])
    random.setstate(state["python"])
    if "cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["cuda"])
    if "numpy" in state:
        import numpy as np
        np.random.set_state(state["numpy"])


def _dcp_save(state: dict, path: str) -> None:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dcp.save(state, checkpoint_id=path)


def _dcp_load(state: dict, path: str) -> None:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        dcp.load(state, checkpoint_id=path)


def whole_parameters(optimizer, writeback: bool = False):
    """With FULL_SHARD the layers' parameters live in rotating working buffers; inside this block they are all whole
    (and, with ``writeback``, what the block wrote becomes the new shards).  A no-op for the other strategies."""
    import contextlib
    block = getattr(optimizer, "full_parameters", None)
    return block(writeback=writeback) if block is not None else contextlib.nullcontext()


def _optimizer_state(optimizer) -> dict:
    sd = optimizer.state_dict()
    flat = {"step": torch.tensor(sd["step"])}
    for group in ("master", "exp_avg", "exp_avg_sq"):
        for name, t in sd[group].items():
            flat[f"{group}.{name}"] = t
    return flat


def save(*, output_dir: str, step_id: int, model: torch.nn.Module, optimizer, draft_config, topology: dict,
         global_step: int, extra_meta: Optional[dict] = None) -> str:
    """Phase one: every rank stages its shards under ``.iter_N.incomplete``."""
    stage = iteration_dir(output_dir, step_id, staging=True)
    if _rank() == 0:
        if os.path.isdir(stage):
            shutil.rmtree(stage)
        os.makedirs(os.path.join(stage, "rng"), exist_ok=True)
    if _world() > 1:
        dist.barrier()
    os.makedirs(os.path.join(stage, "rng"), exist_ok=True)
    with whole_parameters(optimizer):
        model_state = {k: v for k, v in model.state_dict().items()}
        _dcp_save({"model_state": model_state}, os.path.join(stage, "model"))
    _dcp_save({"optim_state": _optimizer_state(optimizer)}, os.path.join(stage, "optimizer"))
    _dcp_save({"lr_scheduler": {"last_epoch": torch.tensor(optimizer.scheduler.last_epoch)}},
              os.path.join(stage, "lr_scheduler"))
    torch.save(_rng_state(), os.path.join(stage, "rng", f"rank-{_rank():05d}.pt"))
    if _rank() == 0:
        meta = {"iteration": int(step_id), "step": int(step_id) - 1, "next_step": int(step_id),
                "global_step": int(global_step), "world_size": _world(), "training_topology": topology,
                "timestamp": time.time(), **(extra_meta or {})}
        with open(os.path.join(stage, "meta.json"), "w") as f:
            json.dump(meta, f, indent=2, sort_keys=True, default=str)
        with open(os.path.join(stage, "draft_config.json"), "w") as f:
            json.dump(draft_config.to_dict() if hasattr(draft_config, "to_dict") else dict(draft_config), f,
                      indent=2, sort_keys=True)
    if _world() > 1:
        dist.barrier()
    return stage


def required_files(stage: str, world_size: int):
    need = [os.path.join(stage, "model", ".metadata"), os.path.join(stage, "optimizer", ".metadata"),
            os.path.join(stage, "lr_scheduler", ".metadata"), os.path.join(stage, "meta.json"),
            os.path.join(stage, "draft_config.json"), os.path.join(stage, "work_state.json")]
    need += [os.path.join(stage, "rng", f"rank-{r:05d}.pt") for r in range(world_size)]
    return need


def publish(*, output_dir: str, step_id: int, work_state: dict, world_size: Optional[int] = None) -> str:
    """Phase two (driver, after the optimizer step is committed): complete and publish atomically."""
    stage = iteration_dir(output_dir, step_id, staging=True)
    final = iteration_dir(output_dir, step_id)
    if not os.path.isdir(stage):
        raise FileNotFoundError(f"no staged checkpoint at {stage}")
    ws = {"schema": WORK_SCHEMA, "optimizer_step": int(step_id) - 1, **work_state}
    with open(os.path.join(stage, "work_state.json"), "w") as f:
        json.dump(ws, f, indent=2, sort_keys=True)
    world_size = world_size or json.load(open(os.path.join(stage, "meta.json")))["world_size"]
    missing = [p for p in required_files(stage, world_size) if not os.path.exists(p)]
    if missing:
        raise RuntimeError("checkpoint is incomplete, refusing to publish: " + ", ".join(os.path.relpath(m, stage) for m in missing))
    with open(os.path.join(stage, "complete.json"), "w") as f:
        json.dump({"schema": COMPLETE_SCHEMA, "iteration": int(step_id), "world_size": world_size,
                   "files": sorted(os.path.relpath(p, stage) for p in required_files(stage, world_size)),
                   "timestamp": time.time()}, f, indent=2, sort_keys=True)
    if os.path.isdir(final):
        shutil.rmtree(final)
    os.replace(stage, final)
    tracker = os.path.join(output_dir, "checkpoints", TRACKER)
    tmp = tracker + ".tmp"
    with open(tmp, "w") as f:
        f.write(str(int(step_id)))
    os.replace(tmp, tracker)
    return final


def latest_iteration(output_dir: str) -> Optional[int]:
    tracker = os.path.join(output_dir, "checkpoints", TRACKER)
    if not os.path.isfile(tracker):
        return None
    return int(open(tracker).read().strip())


def resolve_checkpoint_dir(load_path: str) -> str:
    """Accepts a run dir, its ``checkpoints`` dir or one ``iter_N`` dir."""
    if os.path.isfile(os.path.join(load_path, "complete.json")):
        return load_path
    for root in (load_path, os.path.join(load_path, "checkpoints")):
        tracker = os.path.join(root, TRACKER)
        if os.path.isfile(tracker):
            return os.path.join(root, f"iter_{int(open(tracker).read().strip()):07d}")
    raise FileNotFoundError(f"no complete checkpoint under {load_path}")


def load(*, load_path: str, model: torch.nn.Module, optimizer=None, topology: Optional[dict] = None,
         continual_training: bool = False) -> dict:
    """Loads weights (+ optimizer, scheduler unless ``continual_training``).  RNG is restored by
    ``finalize_load`` so that nothing between here and the first step perturbs it."""
    ckpt = resolve_checkpoint_dir(load_path)
    if not os.path.isfile(os.path.join(ckpt, "complete.json")):
        raise RuntimeError(f"{ckpt} has no complete.json: refusing an incomplete checkpoint")
    meta = json.load(open(os.path.join(ckpt, "meta.json")))
    if not continual_training and topology is not None:
        if meta.get("world_size") != topology.get("world_size"):
            raise ValueError(f"Exact resume refused: world size {topology.get('world_size')} != checkpoint {meta.get('world_size')}")
        validate_exact_resume_topology(meta.get("training_topology", {}), topology)
    with whole_parameters(optimizer, writeback=True):
        state = {"model_state": {k: torch.empty_like(v) for k, v in model.state_dict().items()}}
        _dcp_load(state, os.path.join(ckpt, "model"))
        model.load_state_dict(state["model_state"], strict=True)
    if optimizer is not None:
        if continual_training:
            optimizer.sync_fp32_params_from_model()
        else:
            want = {k: torch.empty_like(v) for k, v in _optimizer_state(optimizer).items()}
            holder = {"optim_state": want}
            _dcp_load(holder, os.path.join(ckpt, "optimizer"))
            got = holder["optim_state"]
            sd = {"step": int(got["step"]), "master": {}, "exp_avg": {}, "exp_avg_sq": {}}
            for key, t in got.items():
                if key == "step":
                    continue
                group, name = key.split(".", 1)
                sd[group][name] = t
            optimizer.load_state_dict(sd)
            sched = {"lr_scheduler": {"last_epoch": torch.tensor(0)}}
            _dcp_load(sched, os.path.join(ckpt, "lr_scheduler"))
            optimizer.scheduler.load_state_dict({"last_epoch": int(sched["lr_scheduler"]["last_epoch"])})
    work_state = json.load(open(os.path.join(ckpt, "work_state.json")))
    return {"checkpoint_dir": ckpt, "meta": meta, "work_state": work_state,
            "next_step": 0 if continual_training else int(meta["next_step"]),
            "global_step": 0 if continual_training else int(meta["global_step"])}


def finalize_load(checkpoint_dir: str) -> None:
    """Restore this rank's RNG streams last (exact resume)."""
    path = os.path.join(checkpoint_dir, "rng", f"rank-{_rank():05d}.pt")
    _restore_rng(torch.load(path, weights_only=False))


def rotate(output_dir: str, keep_last: int, protect: Optional[set] = None) -> list:
    """Delete all but the newest ``keep_last`` complete checkpoints (never those in ``protect``)."""
    root = os.path.join(output_dir, "checkpoints")
    if keep_last <= 0 or not os.path.isdir(root):
        return []
    its = sorted(int(n[5:]) for n in os.listdir(root) if n.startswith("iter_") and n[5:].isdigit())
    doomed = [i for i in its[:-keep_last] if i not in (protect or set())]
    for i in doomed:
        shutil.rmtree(os.path.join(root, f"iter_{i:07d}"), ignore_errors=True)
    return doomed
