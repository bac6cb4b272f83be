"""The driver's training loop: plan -> produce -> train -> commit -> log / evaluate / checkpoint.

One optimizer step has a single wall-clock budget covering supply, transfer, compute and commit
(``optimizer_step_timeout_seconds``); when it runs out the step fails with ``TrainerStepTimeoutError`` and
the driver terminates the trainer processes instead of waiting on a native call
(reference: aspec/controller/loop.py:154-220, 1329-2276).  Rows for step ``s + 1`` are submitted while the
trainers work on step ``s`` (dispatch-ahead, bounded by the ring slots).
"""
from __future__ import annotations

import os
import time
from typing import Callable, Dict, List, Optional

from aspec_b200.runtime.actor import ActorError
from aspec_b200.training import checkpoint as ckpt


class TrainerStepTimeoutError(TimeoutError):
    pass


class ThroughputWindow:
    """Steady-window accounting: starts when warm-up update W completes, ends at the last optimizer
    completion, counts only tokens committed inside (reference: docs/benchmarks/methodology.md:29-36)."""

    def __init__(self, warmup_steps: int = 0, drain_steps: int = 0):
        self.warmup, self.drain = int(warmup_steps), int(drain_steps)
        self.records: List[tuple] = []       # (completed_step_index, t_done, tokens)

    def add(self, step_index: int, tokens: int) -> None:
        self.records.append((step_index, time.perf_counter(), int(tokens)))

    def summary(self) -> dict:
        recs = self.records
        if len(recs) <= self.warmup + self.drain:
            return {"valid": False, "steps": len(recs)}
        start = recs[self.warmup - 1][1] if self.warmup > 0 else None
        body = recs[self.warmup: len(recs) - self.drain] if self.drain else recs[self.warmup:]
        if start is None or not body:
            return {"valid": False, "steps": len(recs)}
        tokens = sum(r[2] for r in body)
        seconds = body[-1][1] - start
        return {"valid": seconds > 0, "steps": len(body), "tokens": tokens, "seconds": seconds,
                "tokens_per_second": tokens / seconds if seconds > 0 else None}


def training_loop(*, controller, manager, trainers, rings, train_queues, args: Dict, layer_ids, num_steps: int,
                  start_step: int = 0, log: Callable[[dict], None] = print, evidence=None, timeline=None,
                  consumer_of_rank: Optional[Callable[[int], List[int]]] = None,
                  on_step: Optional[Callable[[int, dict], None]] = None) -> dict:
    """Runs ``num_steps`` optimizer updates.  ``trainers[r]`` are actors; ``rings[c]`` the lease rings."""
    accumulation = int(args.get("draft_accumulation_steps", 1))
    budget = float(args.get("optimizer_step_timeout_seconds", 1800.0))
    save_interval = int(args.get("save_interval", 0) or 0)
    output_dir = args.get("output_dir") or ""
    dp = controller.dp_size
    consumer_of_rank = consumer_of_rank or (lambda r: [r])
    window = ThroughputWindow(int(args.get("performance_warmup_steps", 0)), int(args.get("performance_drain_steps", 0)))
    results_by_row: Dict[str, tuple] = {}
    submitted_plans: Dict[int, list] = {}
    history: List[dict] = []
    rank_of_row: Dict[str, int] = {}

    def on_result(out, req) -> None:
        # engine finished a row: account for it, then hand one descriptor to each consumer's queue
        from aspec_b200.utils.types import TrainSample
        controller.register_result(out)
        results_by_row[out.row_id] = (out, req)
        for key, (consumer, _slot, _gen) in zip(out.feature_keys, req.leases):
            train_queues[consumer].put(TrainSample(key, out.tensor_shapes, out.document_lengths, out.packed_loss_masks,
                                                   out.metadata, out.data_ids, out.row_id))

    manager.on_result = on_result

    epoch_boundaries: set = set()
    last_saved = None

    def submit(step: int) -> bool:
        plan = controller.plan_update(accumulation)
        if plan is None:
            if int(args.get("num_epochs", 1)) > controller.epoch + 1:
                controller.next_epoch()
                epoch_boundaries.add(step)          # update ``step`` opens an epoch: ``step`` updates complete the last one
                plan = controller.plan_update(accumulation)
            if plan is None:
                return False
        rows = []
        for micro in plan:
            for rank, idxs in enumerate(micro):
                req = controller.row_request(idxs, layer_ids)
                rows.append((rank, req))
                manager.submit(req, consumer_of_rank(rank))
        submitted_plans[step] = rows
        return True

    # how many updates beyond the one in training have their rows at the producers: 1 keeps the Targets one update
    # ahead; a long-context run with one row per update needs as many as there are Target GPUs to keep them all busy
    ahead = max(int(args.get("dispatch_ahead_updates", 1) or 1), 1)
    # train-with-decode: every ``decode_weight_sync_interval`` updates the decoding Target engines reload the live Draft
    sync_every = (int(args.get("decode_weight_sync_interval", 500)) if args.get("train_with_decode")
                  and args.get("decode_weight_sync_enabled") and output_dir and hasattr(manager, "engines") else 0)
    synced = 0
    completed = 0
    step = start_step
    have_next = submit(step)
    submitted_to = step if have_next else step - 1        # last update whose rows were handed to the producers
    exhausted = not have_next
    while have_next and completed < num_steps:
        t_step = time.perf_counter()
        deadline = t_step + budget
        futures = [t.call_async("train_from_queue", step, accumulation, budget) for t in trainers]
        # dispatch-ahead: the producers work on the next update while the trainers compute this one
        while not exhausted and submitted_to < min(step + ahead, start_step + num_steps - 1):
            if submit(submitted_to + 1):
                submitted_to += 1
            else:
                exhausted = True
        have_next = (completed + 1 < num_steps) and submitted_to >= step + 1
        outs = [None] * len(futures)
        pending = set(range(len(futures)))
        while pending:
            # a failed trainer is reported at once (its peers may be blocked in a collective with it)
            for r in sorted(pending):
                if futures[r].done():
                    try:
                        outs[r] = futures[r].get(timeout=1.0)
                    except ActorError:
                        for t in trainers:
                            t.terminate()
                        raise
                    pending.discard(r)
            if not pending:
                break
            manager.raise_if_failed()
            if time.perf_counter() > deadline:
                for t in trainers:
                    t.terminate()
                raise TrainerStepTimeoutError(
                    f"optimizer step {step} exceeded its {budget:.0f}s budget; trainer processes were terminated")
            dead = [r for r in pending if not trainers[r].is_alive()]
            if dead:
                for t in trainers:
                    t.terminate()
                raise ActorError(f"trainer {dead[0]} exited during optimizer step {step}")
            time.sleep(0.02)
        # release leases, then commit the work of this optimizer step
        committed: List[str] = []
        lease_row = {tuple(l): row_id for row_id, (_o, rq) in results_by_row.items() for l in rq.leases}
        trained_rows: Dict[str, List[int]] = {}               # rows this update really consumed -> their readers
        for out in outs:
            for consumer, slot, gen in out["releases"]:
                row_id = lease_row.get((consumer, slot, gen))
                rings[consumer].release_acknowledged(slot, gen, f"row:{row_id or 'unknown'}")
                if row_id is None:
                    raise RuntimeError(f"trainer {consumer} released slot {slot} (generation {gen}) that no reported row leased")
                trained_rows.setdefault(row_id, []).append(consumer)
            committed.extend(out["committed"])
        # with several producers, rows finish in any order: an update trains on the rows that arrived, which need not
        # be the ones planned under its number (the ledger commits what was really consumed)
        submitted_plans.pop(step, None)
        tokens = 0
        decode_stats: Dict[str, int] = {}
        for row_id, consumers in trained_rows.items():
            res, req = results_by_row.pop(row_id)
            for consumer in consumers:                         # every reader of the row releases its own lease
                controller.release_result(res, participant=f"trainer{consumer}")
            tokens += sum(res.document_lengths)              # of the row as produced (a decoding Target lengthens it)
            for k, v in (res.stats or {}).items():
                decode_stats[k] = decode_stats.get(k, 0) + v
        controller.commit_optimizer_step(step, committed)
        completed += 1
        window.add(completed, tokens)
        metrics = dict(outs[0]["metrics"])
        metrics["perf/step_wall_time"] = time.perf_counter() - t_step
        metrics["perf/input_tokens"] = tokens
        metrics["train/step"] = step
        if decode_stats:
            metrics["decode/generated_tokens"] = decode_stats["generated_tokens"]
            metrics["decode/tokens_per_target_pass"] = decode_stats["generated_tokens"] / max(decode_stats["target_passes"], 1)
            if decode_stats.get("verify_rounds"):
                metrics["decode/accepted_draft_tokens_per_round"] = decode_stats["accepted_draft_tokens"] / decode_stats["verify_rounds"]
        history.append(metrics)
        log(metrics)
        if timeline:
            timeline.event("optimizer_step", step=step, tokens=tokens)
        next_step_id = step + 1
        if output_dir and ((save_interval and next_step_id % save_interval == 0)
                           or (args.get("save_per_epoch") and next_step_id in epoch_boundaries)):
            save_checkpoint(trainers, controller, output_dir, next_step_id, args)
            last_saved = next_step_id
        if sync_every and next_step_id % sync_every == 0:
            sync_draft_weights(trainers, manager.engines, os.path.join(output_dir, "scratch_draft_model"), args)
            synced += 1
        if on_step is not None:
            on_step(next_step_id, metrics)          # held-out evaluation, trackers
        step += 1
    if output_dir and args.get("save_final_checkpoint", True) and completed and last_saved != step:
        save_checkpoint(trainers, controller, output_dir, step, args)
    summary = {"completed_steps": completed, "last_step": step - 1, "window": window.summary(),
               "ledger": controller.ledger.status(), "dropped_tail_samples": controller.dropped_tail,
               "history": history}
    if sync_every:
        summary["decode_weight_syncs"] = synced
    return summary


def _owner(results_by_row, consumer, slot, gen) -> str:
    for row_id, (out, req) in results_by_row.items():
        if (consumer, slot, gen) in [tuple(l) for l in req.leases]:
            return f"row:{row_id}"
    return "row:unknown"


def sync_draft_weights(trainers, engines, asset_dir: str, args: Dict) -> None:
    """The trainers write the live Draft as a native asset (rank 0 writes, all ranks join a sharded gather) and every
    Target engine loads it between two of its calls; rows already being decoded finish with the older weights, which
    changes their speed, never their text."""
    timeout = float(args.get("checkpoint_timeout_seconds", 1800.0))
    for fut in [t.call_async("export_draft_asset", asset_dir) for t in trainers]:
        fut.get(timeout=timeout)
    for fut in [e.call_async("load_draft", asset_dir) for e in engines]:
        fut.get(timeout=timeout)


def save_checkpoint(trainers, controller, output_dir: str, step_id: int, args: Dict) -> str:
    """Two-phase: trainers stage their shards, then the driver publishes with the committed work state."""
    for fut in [t.call_async("save_model", output_dir, step_id) for t in trainers]:
        fut.get(timeout=float(args.get("checkpoint_timeout_seconds", 1800.0)))
    final = ckpt.publish(output_dir=output_dir, step_id=step_id, work_state=controller.work_state(),
                         world_size=len(trainers))
    keep = int(args.get("max_checkpoints", 0) or 0)
    if keep:
        ckpt.rotate(output_dir, keep)
    return final
