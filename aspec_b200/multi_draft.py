"""Several Drafts trained from one Target pool ("shared Target, multi-Draft").

``experiments[]`` in the recipe lists Drafts that differ in their model config and hyper-parameters but consume the
same document stream.  Each gets a child execution plan, its own trainer group, optimizer, ledger and checkpoints
under ``<output_dir>/experiments/<name>``; the Target pool runs once per row and its epilogues store into every
experiment's ring slot, each reader keeping only the captured layers it asked for
(reference: aspec/multi_draft.py:51-835; fan-out semantics in aspec/controller/shared_source.py:313-409).

One experiment failing or being cancelled fences its readers; its siblings continue.
"""
from __future__ import annotations

import copy
import dataclasses
import json
import os
import threading
import time
from typing import Any, Dict, List, Optional

from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.config.train_config import Config, _apply, _merge, validate_config
from aspec_b200.feature_contract import build_target_feature_contract, shared_feature_union
from aspec_b200.planning import ExecutionPlan, compile_execution_plan

# what every experiment must share so that all of them plan identical rows
_SHARED_ROW_KEYS = ("train_data_path", "max_seq_length", "micro_batch_size", "draft_accumulation_steps", "dflash_packing",
                    "seed", "dataset_seed", "num_epochs",
                    "synthetic_num_documents", "synthetic_min_length", "synthetic_max_length", "synthetic_vocab_size",
                    # held-out rows are produced once and read by all experiments, at the same updates
                    "eval_data_path", "eval_interval", "eval_num_documents")


@dataclasses.dataclass
class MultiDraftPlan:
    names: List[str]
    plans: Dict[str, ExecutionPlan]
    union: Dict[str, Any]                    # shared feature contract + per-reader views
    consumer_offsets: Dict[str, int]
    schema_version: str = "aspec.multi-draft-plan/v1"
    configs: Dict[str, Config] = dataclasses.field(default_factory=dict)      # every experiment's resolved configuration

    @property
    def plan_id(self) -> str:
        import hashlib
        body = json.dumps({n: self.plans[n].plan_id for n in self.names}, sort_keys=True)
        return "sha256:" + hashlib.sha256(body.encode()).hexdigest()

    def to_json(self) -> str:
        return json.dumps({"schema_version": self.schema_version, "plan_id": self.plan_id, "experiments": self.names,
                           "consumer_offsets": self.consumer_offsets, "shared_feature_contract": self.union["contract"],
                           "reader_views": self.union["views"],
                           "plans": {n: json.loads(p.to_json()) for n, p in self.plans.items()}}, indent=2, default=str)


def _layer_ids(draft: dict) -> List[int]:
    cfg = AutoDraftModelConfig.from_dict(draft)
    ids = list(getattr(cfg, "target_layer_ids", None) or [])
    if not ids:
        from aspec_b200.models.draft.dflash import build_target_layer_ids
        ids = build_target_layer_ids(int(getattr(cfg, "num_target_layers", 3)), int(getattr(cfg, "target_num_hidden_layers", 36)))
    return ids


def _contract(draft: dict) -> dict:
    algorithm = resolve_draft_algorithm(draft)
    return build_target_feature_contract(
        drafter_family=algorithm, target_hidden_size=int(draft.get("target_hidden_size", draft["hidden_size"])),
        target_num_hidden_layers=int(draft.get("target_num_hidden_layers", 36)), aux_hidden_state_layers=_layer_ids(draft),
        store_last_hidden_states=algorithm != "mtp")


def child_config(config: Config, experiment: Dict[str, Any]) -> Config:
    """Base recipe ⊕ the experiment's overrides, rooted at its own output directory."""
    tree = config.to_dict()
    tree["experiments"] = []
    overrides = {k: v for k, v in experiment.items() if k != "name"}
    tree = _merge(tree, copy.deepcopy(overrides))
    tree["output_dir"] = os.path.join(config.output_dir, "experiments", experiment["name"])
    child = Config()
    _apply(child, tree, "")
    validate_config(child)
    return child


def compile_multi_draft_plan(config: Config) -> MultiDraftPlan:
    if len(config.experiments) < 2:
        raise ValueError("a shared-Target run needs at least two experiments")
    plans, names, configs = {}, [], {}
    for exp in config.experiments:
        names.append(exp["name"])
        configs[exp["name"]] = child_config(config, exp)
        plans[exp["name"]] = compile_execution_plan(configs[exp["name"]])
    first = plans[names[0]].runtime_args
    for n in names:
        if plans[n].runtime_args.get("train_with_decode"):
            raise ValueError(f"experiment {n}: training.train_with_decode is a single-Draft mode; a shared-Target run prefills "
                             "recorded responses")
    for n in names[1:]:
        for key in _SHARED_ROW_KEYS:
            if plans[n].runtime_args.get(key) != first.get(key):
                raise ValueError(f"experiments that share a Target must agree on {key}: "
                                 f"{names[0]}={first.get(key)!r}, {n}={plans[n].runtime_args.get(key)!r}")
    # rows are dealt to data-parallel ranks: experiments may shard their rows over different context-parallel degrees (each
    # reads its own views of the one stored row), but all of them must have the same number of data-parallel ranks
    widths = {n: int(plans[n].policy.get("dp_size") or 1) for n in names}
    if len(set(widths.values())) > 1:
        raise ValueError("experiments that share a Target must have the same number of data-parallel ranks "
                         f"(world size / context-parallel size): {widths}")
    union = shared_feature_union([_contract(plans[n].draft_config) for n in names])
    offsets, at = {}, 0
    for n in names:
        offsets[n] = at
        at += int(plans[n].runtime_args["world_size"])
    return MultiDraftPlan(names, plans, union, offsets, configs=configs)


def experiment_load_path(flat: Dict[str, Any], name: str) -> Optional[str]:
    """Where one experiment resumes from.  ``training.load_path`` may name that experiment's own run directory or
    checkpoint, or the root of an earlier shared-Target run (the directory that holds ``experiments/``), in which case
    every experiment takes ``<root>/experiments/<its name>``.  ``{experiment}`` in the path stands for the name, which
    lets one base setting point every experiment at an earlier checkpoint of its own
    (``<root>/experiments/{experiment}/checkpoints/iter_0000100``)."""
    path = flat.get("load_path")
    if not path:
        return None
    path = str(path).replace("{experiment}", name)
    nested = os.path.join(str(path), "experiments", name)
    return nested if os.path.isdir(nested) else str(path)


def _common_samples(controllers: Dict[str, Any], dataset: Optional[List[dict]]) -> List[dict]:
    """Admit a document only if every experiment admits it, so that all of them see the same stream."""
    admitted = None
    for c in controllers.values():
        c.load_dataset(dataset)
        ids = {s["data_id"] for s in c.samples}
        admitted = ids if admitted is None else admitted & ids
    any_c = next(iter(controllers.values()))
    return [s for s in any_c.samples if s["data_id"] in admitted]


def run_multi_draft(plan: MultiDraftPlan, *, dataset: Optional[List[dict]] = None, log=print,
                    cancel: Optional[Dict[str, threading.Event]] = None, claim_directories: bool = True) -> Dict[str, Any]:
    """``claim_directories=False``: the caller has already claimed every experiment's run directory (and keeps their
    evidence)."""
    from aspec_b200.controller.inference_manager import InferenceManager
    from aspec_b200.controller.loop import training_loop
    from aspec_b200.controller.shared_source import SharedSourceState
    from aspec_b200.controller.training_controller import TrainingController
    from aspec_b200.inference.factory import create_engines
    from aspec_b200.runtime.actor import ProcessActor, make_queue
    from aspec_b200.train_entry import _devices, claim_run_directory
    from aspec_b200.training.trainer_actor import TrainerActor
    from aspec_b200.transport.slot_ring import GenerationSlotRing

    names = plan.names
    base = plan.plans[names[0]].to_runtime_args()
    target_devs, _ = _devices(base)
    union_layers = plan.union["contract"]["aux_hidden_state_layers"]
    groups: Dict[str, dict] = {}
    engines: list = []
    manager = None
    results: Dict[str, Any] = {}
    try:
        # ---- one trainer group per experiment --------------------------------------------------------
        next_dev = 0
        for n in names:
            flat = plan.plans[n].to_runtime_args()
            if claim_directories:
                claim_run_directory(flat["output_dir"])
                with open(os.path.join(flat["output_dir"], "plan.json"), "w") as f:
                    f.write(plan.plans[n].to_json())
            world = int(flat["world_size"])
            devs = flat.get("trainer_devices")
            if not devs:
                total = sum(int(plan.plans[m].runtime_args["world_size"]) for m in names)
                _, pool = _devices({**flat, "training_num_gpus_per_node": total, "training_num_nodes": 1})
                devs = pool[next_dev:next_dev + world]
                next_dev += world
            args = dict(flat, trainer_devices=devs, run_id=flat.get("run_id") or f"run-{int(time.time())}-{n}",
                        attempt_id=str(flat.get("attempt_id", "0")))
            port = int(flat.get("master_port") or 29500 + (os.getpid() % 2000)) + 17 * (names.index(n) + 1)
            queues = {r: make_queue() for r in range(world)}
            trainers = [ProcessActor(TrainerActor, r, world, args, plan.plans[n].draft_config, queues[r], port,
                                     name=f"{n}-trainer{r}") for r in range(world)]
            groups[n] = dict(flat=flat, args=args, world=world, queues=queues, trainers=trainers,
                             layer_ids=_layer_ids(plan.plans[n].draft_config))
        for g in groups.values():
            for t in g["trainers"]:
                t.wait_ready()
        # ---- one engine pool: every reader's ring, tagged with the layers it keeps ---------------------
        n_producers = max(len(target_devs), 1)
        handles: Dict[int, list] = {}
        for n in names:
            g = groups[n]
            for r, t in enumerate(g["trainers"]):
                hs = t.call("ring_handle", n_producers, timeout=120)
                for h in hs:
                    h["layer_ids"] = list(g["layer_ids"])
                handles[plan.consumer_offsets[n] + r] = hs
        union_draft = dict(plan.plans[names[0]].draft_config, target_layer_ids=list(union_layers),
                           num_target_layers=len(union_layers))
        engines, head, embedding = create_engines(base, union_draft, list(union_layers), target_devs, handles)
        pick = lambda v, i: v[i] if isinstance(v, list) else v
        for n in names:
            g = groups[n]
            futs = [t.call_async("set_head", pick(head, plan.consumer_offsets[n] + r), pick(embedding, plan.consumer_offsets[n] + r))
                    for r, t in enumerate(g["trainers"])]
            for f in futs:
                f.get(timeout=600)
        # ---- shared stream --------------------------------------------------------------------------------
        slots = int(base.get("transport_destination_ring_slots", 4))
        all_rings: Dict[int, GenerationSlotRing] = {}
        controllers = {}
        for n in names:
            g = groups[n]
            cp = max(int(g["flat"].get("draft_context_parallel_size", 1)), 1)
            g["cp"], g["dp"] = cp, g["world"] // cp
            g["rings"] = {r: GenerationSlotRing(slots) for r in range(g["world"])}
            for r, ring in g["rings"].items():
                all_rings[plan.consumer_offsets[n] + r] = ring
            controllers[n] = TrainingController(g["args"], dp_size=g["dp"], consumers_per_row=cp,
                                                algorithm=resolve_draft_algorithm(plan.plans[n].draft_config))
        common = _common_samples(controllers, dataset)
        own_admission = {n: dict(getattr(c, "admission", None) or {}) for n, c in controllers.items()}
        for c in controllers.values():
            c.load_dataset(common)
        # packed rows are cut by a per-document work measure that depends on the algorithm (anchor starts, TTT positions);
        # readers of one Target pass must cut the same rows, so all of them pack by the first experiment's measure
        work = {s["data_id"]: s["useful"] for s in controllers[names[0]].samples}
        for n in names[1:]:
            for s in controllers[n].samples:
                s["useful"] = work[s["data_id"]]
        # held-out split: the same admission rule (a document every experiment admits), so that all of them ask for the
        # same held-out rows
        eval_controllers = {}
        if base.get("eval_data_path") and int(base.get("eval_interval") or 0) > 0:
            for n in names:
                g = groups[n]
                eval_args = dict(g["args"], train_data_path=g["flat"]["eval_data_path"], shuffle_dataset=False, train_with_decode=False,
                                 synthetic_num_documents=int(g["flat"].get("eval_num_documents") or 32),
                                 dataset_seed=int(g["flat"].get("seed", 0)) + 1)
                eval_controllers[n] = TrainingController(eval_args, dp_size=g["dp"], consumers_per_row=g["cp"],
                                                         algorithm=resolve_draft_algorithm(plan.plans[n].draft_config))
            held_out = _common_samples(eval_controllers, None)
            for ec in eval_controllers.values():
                ec.load_dataset(held_out)
        from aspec_b200.controller.training_controller import draft_vocabulary_from_samples
        for n in names:
            mapping = draft_vocabulary_from_samples(common, plan.plans[n].draft_config, groups[n]["flat"])
            if mapping is not None:
                for fut in [t.call_async("set_vocab_mapping", *mapping) for t in groups[n]["trainers"]]:
                    fut.get(timeout=300)
        # ---- resume: every experiment loads its own checkpoint; readers of one stream must stand at the same row ------
        start_steps = {n: 0 for n in names}
        for n in names:
            g = groups[n]
            load_path = experiment_load_path(g["flat"], n)
            if not load_path:
                continue
            continual = bool(g["flat"].get("continual_training"))
            infos = [f.get(timeout=1800) for f in [t.call_async("load_model", load_path, continual) for t in g["trainers"]]]
            if not continual or g["flat"].get("continue_source_cursor"):
                controllers[n].restore(infos[0]["work_state"])
            start_steps[n] = int(infos[0]["next_step"])
        cursors = {n: (start_steps[n], len(controllers[n].committed_ids)) for n in names}
        if len(set(cursors.values())) > 1:
            raise ValueError("experiments of a shared-Target run must resume from the same update and the same committed rows: "
                             + ", ".join(f"{n}: update {s}, {c} rows" for n, (s, c) in cursors.items()))
        manager = InferenceManager(engines, all_rings, on_result=lambda o, r: None,
                                   batch_size=int(base.get("inference_batch_size", 1)),
                                   acquire_timeout=float(base.get("transport_acquire_timeout_seconds", 120.0)))
        shared = SharedSourceState(manager, names, plan.consumer_offsets)
        manager.start()

        def run_one(n: str) -> None:
            g = groups[n]
            c = controllers[n]
            steps = int(g["flat"].get("num_train_steps") or 0) or max(
                len(c.samples) // max(g["dp"] * int(g["flat"].get("micro_batch_size", 1))
                                      * int(g["flat"].get("draft_accumulation_steps", 1)), 1), 1)
            cp = g["cp"]
            consumer_of_rank = lambda r: list(range(r * cp, (r + 1) * cp))       # noqa: E731
            on_step, runner = None, None
            if n in eval_controllers:
                # held-out evaluation: every experiment asks for the same held-out rows at the same updates; the shared
                # stream produces each row once, and every experiment keeps its own cache, history and best checkpoint
                from aspec_b200.controller.eval import EvalRunner
                runner = EvalRunner(controller=eval_controllers[n], manager=shared.proxy(n), trainers=g["trainers"], rings=g["rings"],
                                    train_queues=g["queues"], args=g["args"], layer_ids=g["layer_ids"],
                                    consumer_of_rank=consumer_of_rank,
                                    decode_anchors_per_doc=int(g["flat"].get("eval_decode_anchors_per_doc") or 0))
                interval = int(g["flat"]["eval_interval"])

                def on_step(next_step: int, metrics: dict, n=n, runner=runner, interval=interval) -> None:
                    if next_step % interval == 0:
                        log({"experiment": n, "train/step": next_step - 1, **runner.run(next_step)})
            try:
                results[n] = training_loop(controller=c, manager=shared.proxy(n), trainers=g["trainers"], rings=g["rings"],
                                           train_queues=g["queues"], args=g["args"], layer_ids=g["layer_ids"],
                                           num_steps=steps - start_steps[n], start_step=start_steps[n],
                                           log=lambda m, n=n: log({"experiment": n, **m}),
                                           consumer_of_rank=consumer_of_rank, on_step=on_step)
                if runner is not None:
                    results[n]["evaluation"] = {"history": runner.history, "best": runner.best}
                # a document is in the shared stream only if every experiment admits it: what this experiment's own rule
                # rejected, and what it lost to its siblings' rules
                own = own_admission[n]
                rejected = dict(own.get("rejected") or {})
                lost = int(own.get("source_rows", len(c.samples))) - sum(rejected.values()) - len(c.samples)
                if lost > 0:
                    rejected["not_admitted_by_every_experiment"] = lost
                results[n]["admission"] = {"admitted": len(c.samples), "source_rows": own.get("source_rows", len(c.samples)),
                                           "rejected": rejected, "fingerprint": c.dataset_fingerprint()}
            except BaseException as exc:                       # noqa: BLE001 - one experiment must not stop the others
                results[n] = {"failed": f"{type(exc).__name__}: {exc}"}
                log({"experiment": n, "failed": results[n]["failed"][:400]})
                shared.fence(n, results[n]["failed"])
                for t in g["trainers"]:
                    t.terminate()

        threads = {n: threading.Thread(target=run_one, args=(n,), name=f"experiment-{n}", daemon=True) for n in names}
        for t in threads.values():
            t.start()
        while any(t.is_alive() for t in threads.values()):
            for n, ev in (cancel or {}).items():
                if ev.is_set() and n in shared.live:
                    shared.fence(n, "cancelled")
                    for t in groups[n]["trainers"]:
                        t.terminate()
            time.sleep(0.05)
        results["shared_source"] = shared.status()
        return results
    finally:
        if manager is not None:
            manager.stop()
        for a in list(engines) + [t for g in groups.values() for t in g["trainers"]]:
            if isinstance(a, ProcessActor):
                a.shutdown(timeout=5.0)


def run_multi_draft_from_config(config: Config, dry_run: bool = False) -> int:
    plan = compile_multi_draft_plan(config)
    if dry_run:
        print(plan.to_json())
        return 0
    os.makedirs(config.output_dir, exist_ok=True)
    with open(os.path.join(config.output_dir, "multi-draft-plan.json"), "w") as f:
        f.write(plan.to_json())
    # every experiment's directory is a run directory of its own (configuration, plan, evidence: ``--report`` works on
    # it); the root keeps the session's evidence (reference: aspec/multi_draft.py:404-440)
    from aspec_b200.config.train_config import save_config
    from aspec_b200.evidence import RunEvidenceRecorder
    from aspec_b200.train_entry import claim_run_directory
    session = {"schema_version": "aspec.multi-draft-evidence/v1", "plan_id": plan.plan_id, "state": "running",
               "started_at": time.time(), "experiments": {}}

    def persist_session() -> None:
        tmp = os.path.join(config.output_dir, "evidence.json.tmp")
        with open(tmp, "w") as f:
            json.dump(session, f, indent=2, sort_keys=True, default=str)
        os.replace(tmp, os.path.join(config.output_dir, "evidence.json"))

    recorders: Dict[str, RunEvidenceRecorder] = {}
    for name in plan.names:
        out_dir = plan.plans[name].runtime_args["output_dir"]
        claim_run_directory(out_dir)
        if name in plan.configs:
            save_config(plan.configs[name], os.path.join(out_dir, "config.yaml"))
        with open(os.path.join(out_dir, "plan.json"), "w") as f:
            f.write(plan.plans[name].to_json())
        recorders[name] = RunEvidenceRecorder(plan.plans[name], out_dir)
        session["experiments"][name] = {"state": "running", "plan_id": plan.plans[name].plan_id, "output_dir": out_dir}
    persist_session()
    # node preflight for the whole session: the Draft GPUs of all experiments plus the shared Target pool
    from aspec_b200.preflight import run_cluster_preflight
    first = plan.plans[plan.names[0]].to_runtime_args()
    pre = run_cluster_preflight(dict(first, world_size=sum(int(p.runtime_args["world_size"]) for p in plan.plans.values()),
                                     output_dir=config.output_dir))
    with open(os.path.join(config.output_dir, "cluster-preflight.json"), "w") as f:
        json.dump(pre, f, indent=2, default=str)
    for rec in recorders.values():
        rec.record_cluster_preflight(pre)
    if pre.get("state") == "failed":
        exc = RuntimeError(f"node preflight failed: {pre['problems']} (details in cluster-preflight.json)")
        for name, rec in recorders.items():
            rec.fail(exc)
            session["experiments"][name]["state"] = "failed"
        session.update(state="failed", finished_at=time.time(), failure=str(exc))
        persist_session()
        raise exc
    from aspec_b200.utils.logging import Trackers
    trackers: Dict[str, Trackers] = {}

    def log(m: dict) -> None:
        """One metrics writer per experiment, under that experiment's own run directory."""
        print(json.dumps(m, default=float), flush=True)
        name = m.get("experiment")
        if name not in plan.plans:
            return
        if name not in trackers:
            flat = plan.plans[name].to_runtime_args()
            wanted = [t for t, key in (("tensorboard", "use_tensorboard"), ("wandb", "use_wandb")) if flat.get(key)]
            os.makedirs(flat["output_dir"], exist_ok=True)
            trackers[name] = Trackers(flat["output_dir"], ",".join(wanted) or "none",
                                      project=flat.get("wandb_project") or "aspec-b200", run_name=f"{flat.get('wandb_run_id') or 'run'}-{name}",
                                      wandb_mode=flat.get("wandb_mode") or "offline", wandb_group=flat.get("wandb_group"),
                            wandb_team=flat.get("wandb_team"), wandb_dir=flat.get("wandb_dir"))
        trackers[name].log({k: v for k, v in m.items() if k != "experiment"}, int(m.get("train/step") or 0))

    try:
        results = run_multi_draft(plan, log=log, claim_directories=False)
    except BaseException as exc:                                   # noqa: BLE001 - recorded, then re-raised
        for name, rec in recorders.items():
            rec.fail(exc)
            session["experiments"][name]["state"] = "failed"
        session.update(state="failed", finished_at=time.time(), failure=f"{type(exc).__name__}: {exc}"[:2000])
        persist_session()
        raise
    finally:
        for t in trackers.values():
            t.close()
    for name, rec in recorders.items():
        res = results.get(name) or {}
        if "failed" in res:
            rec.fail(RuntimeError(res["failed"]))
        else:
            adm = res.get("admission") or {}
            rec.record_dataset_admission(dataset_size=int(adm.get("admitted", 0)), admission=adm)
            rec.complete({k: v for k, v in res.items() if k not in ("history", "admission")})
        session["experiments"][name].update(state="failed" if "failed" in res else "completed",
                                            completed_steps=res.get("completed_steps"), failure=res.get("failed"))
    session.update(state="completed" if all(e["state"] == "completed" for e in session["experiments"].values()) else "failed",
                   finished_at=time.time(), shared_source=results.get("shared_source"))
    persist_session()
    with open(os.path.join(config.output_dir, "multi-draft-summary.json"), "w") as f:
        json.dump({k: ({kk: vv for kk, vv in v.items() if kk != "history"} if isinstance(v, dict) else v)
                   for k, v in results.items()}, f, indent=2, default=str)
    return 0 if all("failed" not in v for k, v in results.items() if k != "shared_source") else 1
