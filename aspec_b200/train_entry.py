"""``aspec --config recipe.yaml``: load and validate the config, compile the plan, start the role
processes and run the training loop (reference: aspec/train_entry.py:148-622).

Process model on one B200 node: the driver (this process, CPU only) owns the controller, the ledger, the
lease rings and the inference manager; each Target GPU and each Draft GPU is a child process
(``runtime.actor.ProcessActor``).  Draft ranks allocate their feature rings and export them; Target ranks
map them and write features directly into them.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from typing import Any, Dict, List, Optional

from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.config.train_config import load_config, save_config
from aspec_b200.runtime.actor import ProcessActor, make_queue
from aspec_b200.transport.slot_ring import GenerationSlotRing

RUN_ARTIFACTS = ("config.yaml", "plan.json", "evidence.json", "evaluation.json", "tracking.json",
                 "cluster-preflight.json", "checkpoints", "runs", "traces", "scratch_draft_model")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="aspec", description="Train a speculative-decoding draft model.")
    ap.add_argument("--config", help="recipe YAML")
    ap.add_argument("--report", metavar="RUN_DIR", help="render the report of a finished run")
    ap.add_argument("--report-format", default="text", choices=["text", "json"])
    ap.add_argument("--dry-run", action="store_true", help="compile the plan and stop")
    ap.add_argument("--print-config-only", action="store_true")
    ap.add_argument("--preflight-only", action="store_true")
    ap.add_argument("overrides", nargs="*", help="section.key=value")
    return ap


def resolve_draft_config(flat: Dict[str, Any]) -> dict:
    path = flat.get("draft_model_config")
    if not path:
        raise ValueError("model.draft_model_config is required")
    from aspec_b200.assets import load_draft_config
    raw = dict(load_draft_config(path))
    raw.update(flat.get("draft_overrides") or {})
    return AutoDraftModelConfig.from_dict(raw).to_dict()


def claim_run_directory(output_dir: str) -> None:
    """A run directory belongs to one run: refuse to reuse one that already holds evidence."""
    os.makedirs(output_dir, exist_ok=True)
    if os.path.exists(os.path.join(output_dir, "evidence.json")):
        raise FileExistsError(f"{output_dir} already contains a run (evidence.json); choose a fresh output_dir")
    for sub in ("checkpoints", "runs", "traces"):
        os.makedirs(os.path.join(output_dir, sub), exist_ok=True)


def _devices(flat: Dict[str, Any]):
    """Device strings of the Target and Draft roles on this node, from the placement policy (``placement_strategy``,
    ``colocate``, ``training_nodes`` / ``inference_nodes``, ``cluster_nodes``)."""
    import torch
    from aspec_b200.placement import cluster_from_args, create_placement
    n_draft = int(flat["training_num_gpus_per_node"]) * int(flat["training_num_nodes"])
    n_target = int(flat["inference_num_gpus"]) if flat["inference_engine_type"] == "native" else 0
    if torch.cuda.is_available() and not flat.get("force_cpu"):
        have = torch.cuda.device_count()
        nodes = cluster_from_args(flat, have)
        args = dict(flat, inference_num_gpus=n_target)
        roles = None if n_target > 0 else {"training"}
        if roles is None and not flat.get("colocate") and len(nodes) == 1 and n_draft + n_target > have:
            raise RuntimeError(f"plan needs {n_target} Target + {n_draft} Draft GPUs, {have} visible")
        placement = create_placement(args, nodes, roles)
        here = str(flat.get("cluster_node_name") or nodes[0].name)
        target, draft = placement.devices_on(here, "inference"), placement.devices_on(here, "training")
        if len(target) != n_target or len(draft) != n_draft:
            raise RuntimeError(f"placement puts {len(target)} Target + {len(draft)} Draft roles on node {here}; this runtime "
                               f"launches one node and the plan needs {n_target} + {n_draft} there")
    else:
        target, draft = ["cpu"] * n_target, ["cpu"] * n_draft
    return target, draft


def train_async_no_generation(flat: Dict[str, Any], draft_config: dict, evidence=None, log=print,
                              dataset: Optional[List[dict]] = None) -> dict:
    """Starts the actors, runs the loop, tears everything down.  Returns the loop summary."""
    from aspec_b200.controller.inference_manager import InferenceManager
    from aspec_b200.controller.loop import training_loop
    from aspec_b200.controller.training_controller import TrainingController
    from aspec_b200.inference.factory import create_engines
    from aspec_b200.training.trainer_actor import TrainerActor
    algorithm = resolve_draft_algorithm(draft_config)
    target_devs, draft_devs = _devices(flat)
    world = len(draft_devs)
    # ranks that must see the same rows: a context-parallel group shares a row's shards, a vocabulary-parallel group
    # shares its supervised rows
    usp = max(int(flat.get("sp_ulysses_size", 1) or 1), 1) * max(int(flat.get("sp_ring_size", 1) or 1), 1)
    cp = max(int(flat.get("draft_context_parallel_size", 1)), 1)
    if algorithm in ("eagle3", "eagle4"):
        cp = max(cp, usp)                  # the planner folds the sequence-parallel degree into the context-parallel size
    cp *= max(int(flat.get("vocab_parallel_size", 1) or 1), 1)
    dp = world // cp
    args = dict(flat)
    args.update(trainer_devices=draft_devs, run_id=flat.get("run_id") or f"run-{int(time.time())}",
                attempt_id=str(flat.get("attempt_id", "0")))
    cfg_obj = AutoDraftModelConfig.from_dict(draft_config)
    layer_ids = list(getattr(cfg_obj, "target_layer_ids", None) or [])
    if not layer_ids:
        from aspec_b200.models.draft.dflash import build_target_layer_ids
        layer_ids = build_target_layer_ids(int(getattr(cfg_obj, "num_target_layers", 3)),
                                           int(getattr(cfg_obj, "target_num_hidden_layers", 36)))
    port = int(flat.get("master_port") or 29500 + (os.getpid() % 2000))
    queues = {r: make_queue() for r in range(world)}
    trainers = [ProcessActor(TrainerActor, r, world, args, draft_config, queues[r], port, name=f"trainer{r}")
                for r in range(world)]
    engines: list = []
    manager = None
    failed = False
    try:
        for t in trainers:
            t.wait_ready()
        n_producers = max(len(target_devs), 1)
        handles = {r: trainers[r].call("ring_handle", n_producers, timeout=120) for r in range(world)}
        engines, head, embedding = create_engines(flat, draft_config, layer_ids, target_devs, handles)
        pick = lambda v, r: v[r] if isinstance(v, list) else v
        for fut in [t.call_async("set_head", pick(head, r), pick(embedding, r)) for r, t in enumerate(trainers)]:
            fut.get(timeout=600)
        if flat.get("train_with_decode") and flat.get("decode_speculative_draft_model_path"):
            # the decoding Targets start with this exported Draft; weight syncs replace it with the live one later
            for fut in [e.call_async("load_draft", flat["decode_speculative_draft_model_path"]) for e in engines]:
                fut.get(timeout=600)
        start_step = 0
        controller = TrainingController(args, dp_size=dp, consumers_per_row=cp, algorithm=algorithm)
        n = controller.load_dataset(dataset)
        from aspec_b200.controller.training_controller import draft_vocabulary_from_samples
        mapping = draft_vocabulary_from_samples(controller.samples, draft_config, flat)
        if mapping is not None:                      # pruned Draft head: the tokens it predicts come from the corpus
            for fut in [t.call_async("set_vocab_mapping", *mapping) for t in trainers]:
                fut.get(timeout=300)
        if evidence:
            stats = getattr(controller, "admission", None) or {}
            evidence.record_dataset_admission(dataset_size=n, admission={"admitted": n, "fingerprint": controller.dataset_fingerprint(),
                                                                         **stats})
            evidence.record_actor_initialization(
                training_actors=[{"name": f"trainer{r}", "device": str(draft_devs[r]), "pid": getattr(t, "pid", None)}
                                 for r, t in enumerate(trainers)],
                # one entry per engine PROCESS: a tensor-parallel engine has one per GPU it spans
                inference_engines=[{"name": getattr(m, "name", f"engine{i}"), "device": str(target_devs[i]) if i < len(target_devs) else "cpu",
                                    "pid": getattr(m, "pid", None)}
                                   for i, m in enumerate(m for e in engines for m in getattr(e, "members", [e]))])
        if flat.get("load_path"):
            # collective inside the trainer group: start it on every rank before waiting for any
            futs = [t.call_async("load_model", flat["load_path"], bool(flat.get("continual_training"))) for t in trainers]
            infos = [f.get(timeout=1800) for f in futs]
            if not flat.get("continual_training") or flat.get("continue_source_cursor"):
                controller.restore(infos[0]["work_state"])
            start_step = infos[0]["next_step"]
        slots = int(flat.get("transport_destination_ring_slots", 4))
        rings = {r: GenerationSlotRing(slots) for r in range(world)}
        manager = InferenceManager(engines, rings, on_result=lambda o, r: None,
                                   batch_size=int(flat.get("inference_batch_size", 1)),
                                   batch_tokens=int(flat.get("inference_batch_tokens", 0) or 0),
                                   acquire_timeout=float(flat.get("transport_acquire_timeout_seconds", 120.0)))
        manager.start()
        num_steps = int(flat.get("num_train_steps") or 0) or max(n // max(dp * int(flat.get("micro_batch_size", 1))
                                                                     * int(flat.get("draft_accumulation_steps", 1)), 1), 1)
        consumer_of_rank = (lambda r: list(range(r * cp, (r + 1) * cp)))
        on_step = None
        eval_history: list = []
        if flat.get("eval_data_path") and int(flat.get("eval_interval") or 0) > 0:
            from aspec_b200.controller.eval import EvalRunner
            # held-out rows are prefilled with their recorded responses even when training decodes its own
            eval_args = dict(args, train_data_path=flat["eval_data_path"], shuffle_dataset=False, train_with_decode=False,
                             synthetic_num_documents=int(flat.get("eval_num_documents") or 32),
                             dataset_seed=int(flat.get("seed", 0)) + 1)
            eval_controller = TrainingController(eval_args, dp_size=dp, consumers_per_row=cp, algorithm=algorithm)
            eval_controller.load_dataset(None)
            runner = EvalRunner(controller=eval_controller, manager=manager, trainers=trainers, rings=rings, train_queues=queues,
                                args=args, layer_ids=layer_ids, consumer_of_rank=consumer_of_rank,
                                decode_anchors_per_doc=int(flat.get("eval_decode_anchors_per_doc") or 0))
            interval = int(flat["eval_interval"])

            def on_step(next_step: int, metrics: dict) -> None:
                if next_step % interval == 0:
                    m = runner.run(next_step)
                    eval_history.append({"step": next_step, **m})
                    log({"train/step": next_step - 1, **m})
        from aspec_b200.utils.timeline import Timeline
        timeline = Timeline((flat.get("timeline_output_dir") or os.path.join(str(flat.get("output_dir") or "."), "timeline"))
                            if flat.get("timeline_enabled") else None, role="driver", run_id=str(flat.get("timeline_run_id") or ""),
                            flush_every=int(flat.get("timeline_flush_every") or 128), enabled=bool(flat.get("timeline_enabled")))
        try:
            summary = training_loop(controller=controller, manager=manager, trainers=trainers, rings=rings,
                                    train_queues=queues, args=args, layer_ids=layer_ids, num_steps=num_steps - start_step,
                                    start_step=start_step, log=log, evidence=evidence, consumer_of_rank=consumer_of_rank,
                                    on_step=on_step, timeline=timeline)
        finally:
            timeline.close()
        if eval_history:
            summary["evaluation"] = eval_history
        # what rank 0 really launched, beside the plan's capability decisions
        summary["capabilities_observed"] = trainers[0].call("observed_capabilities", timeout=60)
        if evidence:
            for subsystem, counts in summary["capabilities_observed"].items():
                evidence.observe_capability(subsystem, counts)
        traces = [f.get(timeout=300) for f in [t.call_async("flush_debug") for t in trainers]]
        if any(traces):
            summary["trace_files"] = sorted(p for files in traces for p in files)
        summary["engines"] = [e.call("get_status", timeout=30) if isinstance(e, ProcessActor) else e.get_status()
                              for e in engines]
        return summary
    except BaseException:
        failed = True
        raise
    finally:
        # Ownership fence: engine processes store into rings that live in the trainers' memory, so engines are
        # stopped and observed dead before any trainer (the owner of that memory) is allowed to exit.
        from aspec_b200.owner_fence import SourceFence
        if manager is not None:
            manager.stop()
        fence = SourceFence(grace_seconds=5.0, hold_seconds=float(flat.get("fence_hold_seconds", 60.0)),
                            log=lambda msg: print(msg, flush=True))
        for e in engines:
            if isinstance(e, ProcessActor):
                fence.add_accessor(e)
        for t in trainers:
            fence.add_owner(t)
        fence.close(failed=failed)


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.report:
        from aspec_b200.reporting import build_run_report, render_report
        report = build_run_report(a.report)
        print(json.dumps(report, indent=2, default=str) if a.report_format == "json" else render_report(report))
        return 0 if report.get("valid", False) else 1
    if not a.config:
        build_parser().error("--config is required")
    config = load_config(a.config, a.overrides)
    if a.print_config_only:
        import yaml
        print(yaml.safe_dump(config.to_dict(), sort_keys=True))
        return 0
    if config.experiments:
        from aspec_b200.multi_draft import run_multi_draft_from_config
        return run_multi_draft_from_config(config, dry_run=a.dry_run)
    from aspec_b200.evidence import RunEvidenceRecorder
    from aspec_b200.planning import compile_execution_plan
    plan = compile_execution_plan(config)
    if a.dry_run:
        print(plan.to_json())
        return 0
    flat = plan.to_runtime_args()
    claim_run_directory(flat["output_dir"])
    save_config(config, os.path.join(flat["output_dir"], "config.yaml"))
    with open(os.path.join(flat["output_dir"], "plan.json"), "w") as f:
        f.write(plan.to_json())
    evidence = RunEvidenceRecorder(plan, flat["output_dir"])
    try:
        from aspec_b200.preflight import run_cluster_preflight
        pre = run_cluster_preflight(flat)
        with open(os.path.join(flat["output_dir"], "cluster-preflight.json"), "w") as f:
            json.dump(pre, f, indent=2, default=str)
        if pre.get("state") == "failed":
            raise RuntimeError(f"node preflight failed: {pre['problems']} (details in cluster-preflight.json)")
        evidence.record_cluster_preflight(pre)
        if a.preflight_only:
            evidence.complete({"preflight_only": True})
            return 0
        from aspec_b200.utils.logging import Trackers
        wanted = [name for name, key in (("tensorboard", "use_tensorboard"), ("wandb", "use_wandb")) if flat.get(key)]
        trackers = Trackers(flat["output_dir"], ",".join(wanted) or "none", project=flat.get("wandb_project") or "aspec-b200",
                            run_name=flat.get("wandb_run_id"), config=config.to_dict(),
                            wandb_mode=flat.get("wandb_mode") or "offline", wandb_group=flat.get("wandb_group"),
                            wandb_team=flat.get("wandb_team"), wandb_dir=flat.get("wandb_dir"))

        def log(m: dict) -> None:
            trackers.log(m, int(m.get("train/step") or 0))
            print(f"step {m.get('train/step')}: loss {m.get('train/avg_loss', float('nan')):.4f} "
                  f"acc {m.get('train/avg_acc', 0):.3f} tokens {m.get('perf/input_tokens')} "
                  f"wall {m.get('perf/step_wall_time', 0):.3f}s", flush=True)

        try:
            summary = train_async_no_generation(flat, plan.draft_config, evidence, log)
        finally:
            trackers.close()
        evidence.complete({k: v for k, v in summary.items() if k != "history"})
    except BaseException as exc:                                  # noqa: BLE001 - recorded, then re-raised
        evidence.fail(exc)
        raise
    if flat.get("performance_measurement_required") and not (summary.get("window") or {}).get("valid"):
        # the run itself is complete and recorded; what is refused is calling it a throughput measurement
        raise ValueError("debug.performance_measurement_required: the run has no valid steady throughput window "
                         "(needs more optimizer steps than performance_warmup_steps + performance_drain_steps, "
                         "and at least one warm-up step)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
