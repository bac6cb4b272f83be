"""Held-out evaluation inside a training run: every ``eval_interval`` optimizer steps the eval split goes through
the same producer -> ring -> trainer path as training, without gradients; the trainers keep the eval batches in host
memory under an identity (dataset fingerprint + feature contract + row shape), so later evaluations replay from that
cache and need no Target time.  Results append to ``evaluation.json``; the best checkpoint so far is recorded next to
it (reference: aspec/controller/eval.py:42-357)."""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import Any, Callable, Dict, List, Optional


def eval_cache_identity(fingerprint: str, contract_id: str, args: Dict[str, Any]) -> str:
    body = {"dataset": fingerprint, "contract": contract_id, "max_seq_length": args.get("max_seq_length"),
            "micro_batch": args.get("eval_micro_batch_size") or args.get("micro_batch_size", 1),
            "block": args.get("dspark_block_size") or args.get("dflash_block_size"), "seed": args.get("seed", 0)}
    return hashlib.sha256(json.dumps(body, sort_keys=True, default=str).encode()).hexdigest()


class EvalRunner:
    def __init__(self, *, controller, manager, trainers, rings, train_queues, args: Dict[str, Any], layer_ids,
                 contract_id: str = "", consumer_of_rank: Optional[Callable[[int], List[int]]] = None, metric: str = "eval/avg_loss",
                 higher_is_better: bool = False, decode_anchors_per_doc: int = 0):
        self.controller, self.manager, self.trainers, self.rings, self.queues = controller, manager, trainers, rings, train_queues
        self.args, self.layer_ids = args, layer_ids
        self.consumer_of_rank = consumer_of_rank or (lambda r: [r])
        self.identity = eval_cache_identity(controller.dataset_fingerprint(), contract_id, args)
        self.metric, self.higher = metric, higher_is_better
        self.decode_anchors = int(decode_anchors_per_doc)
        self.cached = False
        self.history: List[dict] = []
        self.best: Optional[dict] = None
        self.output_dir = args.get("output_dir") or ""

    def _rows(self) -> List[List[int]]:
        """Deterministic rows: the eval samples in order, one per rank per micro-step (tail dropped evenly)."""
        n, dp = len(self.controller.samples), self.controller.dp_size
        per_rank = n // dp
        return [[r * per_rank + i for r in range(dp)] for i in range(per_rank)]

    def run(self, step: int, checkpoint: Optional[str] = None) -> Dict[str, float]:
        t0 = time.perf_counter()
        if self.cached:
            outs = [f.get(timeout=3600) for f in [t.call_async("eval_from_cache", self.identity) for t in self.trainers]]
            if any(o.get("miss") for o in outs):
                self.cached = False
        if not self.cached:
            rows = self._rows()
            results = {}
            prev = self.manager.on_result

            def on_result(out, req):
                from aspec_b200.utils.types import TrainSample
                if not str(out.row_id).startswith("eval-"):
                    return prev(out, req)              # a dispatched-ahead training row finished during the evaluation
                results[out.row_id] = (out, req)
                for key, (consumer, _s, _g) in zip(out.feature_keys, req.leases):
                    self.queues[consumer].put(TrainSample(key, out.tensor_shapes, out.document_lengths, out.packed_loss_masks,
                                                          out.metadata, out.data_ids, out.row_id))

            self.manager.on_result = on_result
            try:
                for f in [t.call_async("eval_begin", self.identity) for t in self.trainers]:
                    f.get(timeout=600)
                # one row per rank at a time: the trainers hand each lease back right away, so the evaluation fits in the
                # ring slots that the dispatched-ahead training rows leave free
                for micro in rows:
                    futs = [t.call_async("eval_step", 1) for t in self.trainers]
                    for rank, idx in enumerate(micro):
                        req = self.controller.row_request([idx], self.layer_ids)
                        req.row_id = "eval-" + req.row_id
                        self.manager.submit(req, self.consumer_of_rank(rank))
                    for f in futs:
                        for consumer, slot, gen in f.get(timeout=3600)["releases"]:
                            owner = next((f"row:{rid}" for rid, (_o, rq) in results.items()
                                          if (consumer, slot, gen) in [tuple(l) for l in rq.leases]), "row:unknown")
                            self.rings[consumer].release_acknowledged(slot, gen, owner)
                outs = [f.get(timeout=3600) for f in [t.call_async("eval_end") for t in self.trainers]]
                self.cached = all(o.get("cached", 0) == len(rows) for o in outs)
            finally:
                self.manager.on_result = prev
        metrics = dict(outs[0]["metrics"])
        if self.decode_anchors > 0 and self.cached:
            # train-with-decode: block proposals of the live weights on the cached held-out rows (rank 0's share)
            dec = self.trainers[0].call("decode_from_cache", self.identity, self.decode_anchors, timeout=3600).get("decode")
            if dec and dec.get("proposals"):
                metrics.update({"eval/decode_tau": dec["tau"], "eval/decode_fully_accepted": dec["fully_accepted_share"],
                                "eval/decode_proposals": dec["proposals"]})
        record = {"step": step, "seconds": round(time.perf_counter() - t0, 3), "from_cache": bool(self.cached and self.history),
                  "metrics": metrics, "checkpoint": checkpoint}
        self.history.append(record)
        value = metrics.get(self.metric)
        if value is not None and (self.best is None or (value > self.best["value"] if self.higher else value < self.best["value"])):
            self.best = {"step": step, "metric": self.metric, "value": value, "checkpoint": checkpoint}
        if self.output_dir:
            with open(os.path.join(self.output_dir, "evaluation.json"), "w") as f:
                json.dump({"identity": self.identity, "history": self.history, "best": self.best}, f, indent=2, default=float)
        return metrics
