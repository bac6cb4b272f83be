"""Single-process-per-GPU Draft trainer: micro-batch loop, loss pooling, optimizer step, metrics.

What one optimizer update does (reference: aspec/training/trainer.py:641-760,
aspec/training/dflash_trainer.py:489-533, 747-806):

1. for each of ``accumulation`` micro-batches: forward the training wrapper, ``backward`` the raw loss
   *numerator* (weight gradients accumulate in fp32 ``main_grad`` buffers);
2. after the last one: SUM-reduce the flat gradient and the pooled denominators over the data-parallel
   group, and fold ``1 / denominator`` into the optimizer's gradient scale - equivalent to the
   reference's "rescale by world * accumulation / denominator after a mean reduction", without touching
   the gradients twice;
3. fused norm / clip / non-finite skip / AdamW / bf16 write-back; scheduler step; router-bias hooks.

Loss components travel as ``(numerator, denominator)`` pairs and are pooled on the device; ``metrics()``
performs the single device->host read of an update.
"""
from __future__ import annotations

import time
from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

from aspec_b200.training.optimizer import BF16Optimizer

_BATCH_TENSOR_KEYS = ("input_ids", "hidden_states", "loss_mask", "last_hidden_states", "attention_mask",
                      "ctx_doc_ids", "base_position_ids", "packed_context_positions",
                      "injected_anchors", "injected_keep_mask")


# anchors sampled by the data pipeline stay on the host: the block layout is compacted there
_HOST_KEYS = ("injected_anchors", "injected_keep_mask")


class _PhaseClock:
    """Where an update's time goes, without a host synchronisation of its own: phase boundaries are CUDA events on the
    compute stream (host clock on the CPU) and are read when the update's metrics are fetched, which synchronises anyway.
    ``perf/data_time`` is host time spent waiting for rows; the others are device time
    (reference: the perf/* metrics of aspec/training/trainer.py:118-128)."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.reset()

    def reset(self) -> None:
        self.spans: List[tuple] = []
        self.host: Dict[str, float] = {}

    def now(self):
        if not self.cuda:
            return time.perf_counter()
        e = torch.cuda.Event(enable_timing=True)
        e.record(torch.cuda.current_stream(self.device))
        return e

    def span(self, name: str, start, end) -> None:
        self.spans.append((name, start, end))

    def add_host(self, name: str, seconds: float) -> None:
        self.host[name] = self.host.get(name, 0.0) + seconds

    def totals(self) -> Dict[str, float]:
        """Seconds per phase; call only after the stream has been synchronised."""
        out = dict(self.host)
        for name, a, b in self.spans:
            out[name] = out.get(name, 0.0) + (a.elapsed_time(b) / 1e3 if self.cuda else b - a)
        return out


class DraftTrainer:
    def __init__(self, model: torch.nn.Module, lm_head_weight: torch.Tensor, *, lr: float = 6e-4,
                 min_lr: float = 6e-5, weight_decay: float = 0.0, max_grad_norm: float = 1.0,
                 total_steps: int = 1000, warmup_ratio: float = 0.04, decay_style: str = "cosine",
                 accumulation: int = 1, dp_group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None, betas=(0.9, 0.999), fsdp_strategy: str = "REPLICATE",
                 wsd_decay_steps: Optional[int] = None, wsd_decay_style: Optional[str] = None):
        self.model = model
        self.draft = model.draft_model
        self.lm_head_weight = lm_head_weight
        self.accumulation = int(accumulation)
        self.dp_group = dp_group
        self.device = device or next(model.parameters()).device
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(dp_group) > 1
        strategy = str(fsdp_strategy).upper()
        self.sharded = strategy in ("FULL_SHARD", "SHARD_OPTIMIZER") and multi
        if strategy == "FULL_SHARD" and multi:
            # parameters, gradients, masters and moments sharded; layers are gathered for their forward and backward and
            # each layer's gradient is reduce-scattered under the backward of the layers below it
            from aspec_b200.training.full_shard import FullShardOptimizer
            layers = list(getattr(self.draft, "layers", None) or [])
            self.optimizer = FullShardOptimizer(self.draft, layers, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                                                total_steps=total_steps, warmup_ratio=warmup_ratio, decay_style=decay_style,
                                                min_lr=min_lr, betas=betas, group=dp_group,
                                                wsd_decay_steps=wsd_decay_steps, wsd_decay_style=wsd_decay_style)
        elif self.sharded:
            # whole replicas; masters and moments sharded; reduction and update over peer memory once per update
            from aspec_b200.training.sharded_optimizer import ShardedBF16Optimizer
            self.optimizer = ShardedBF16Optimizer(self.draft, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm,
                                                  total_steps=total_steps, warmup_ratio=warmup_ratio, decay_style=decay_style,
                                                  min_lr=min_lr, betas=betas, group=dp_group,
                                                  wsd_decay_steps=wsd_decay_steps, wsd_decay_style=wsd_decay_style)
        else:
            self.optimizer = BF16Optimizer(self.draft, lr=lr, weight_decay=weight_decay,
                                           max_grad_norm=max_grad_norm, total_steps=total_steps,
                                           warmup_ratio=warmup_ratio, decay_style=decay_style, min_lr=min_lr,
                                           betas=betas, wsd_decay_steps=wsd_decay_steps, wsd_decay_style=wsd_decay_style)
        self.global_step = 0
        self.expert_replica_group = None     # set with expert parallelism: ranks that hold the same experts
        self._pool: Dict[str, List[torch.Tensor]] = {}
        self._last: Dict[str, torch.Tensor] = {}
        self.post_step_hooks = []
        self.clock = _PhaseClock(self.device)
        self.pre_step_hooks: list = []
        self._copy_stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    # -- host -> device -------------------------------------------------------------
    def to_device(self, batch: dict) -> dict:
        """Copy a host batch (ideally pinned) to the device; tensors already there pass through."""
        out = {}
        for k, v in batch.items():
            if torch.is_tensor(v) and k in _BATCH_TENSOR_KEYS and k not in _HOST_KEYS:
                out[k] = v.to(self.device, non_blocking=True)
            else:
                out[k] = v
        return out

    def _stage(self, batch):
        """``(device batch, event or None)``: host tensors are copied on a side stream so that the copy of micro-batch
        ``i + 1`` overlaps the compute of micro-batch ``i``; the event marks the end of the copies."""
        if batch is None:
            return None
        if self.device.type != "cuda" or self.h2d_bytes(batch) == 0:
            return self.to_device(batch), None
        if getattr(self, "_copy_stream", None) is None:
            self._copy_stream = torch.cuda.Stream(self.device)
        compute = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self._copy_stream):
            out = self.to_device(batch)
            for k, v in out.items():
                if torch.is_tensor(v) and v.is_cuda and v is not batch.get(k):
                    v.record_stream(compute)              # allocated on the copy stream, consumed on the compute stream
            ready = torch.cuda.Event()
            ready.record(self._copy_stream)
        return out, ready

    @staticmethod
    def h2d_bytes(batch: dict) -> int:
        return sum(v.numel() * v.element_size() for k, v in batch.items()
                   if torch.is_tensor(v) and k in _BATCH_TENSOR_KEYS and not v.is_cuda and k not in _HOST_KEYS)

    # -- one micro-batch ----------------------------------------------------------------
    def _forward_backward(self, batch: dict) -> None:
        t0 = self.clock.now()
        out = self.model(
            batch["input_ids"], batch["hidden_states"], batch["loss_mask"], self.lm_head_weight,
            last_hidden_states=batch.get("last_hidden_states"), ctx_doc_ids=batch.get("ctx_doc_ids"),
            base_position_ids=batch.get("base_position_ids"),
            packed_context_positions=batch.get("packed_context_positions"),
            injected_anchors=batch.get("injected_anchors"),
            injected_keep_mask=batch.get("injected_keep_mask"),
            packed_document_lengths=batch.get("packed_document_lengths"),
            attention_mask=batch.get("attention_mask"))
        loss, acc, loss_pp, acc_pp, count_pp, comps, (num, den) = out
        if num.requires_grad:
            t1 = self.clock.now()
            num.backward()
            close = getattr(self.optimizer, "finish_micro_batch", None)
            if close is not None:            # FULL_SHARD: the root unit's gradients join the reduce-scatter here
                close()
            self.clock.span("forward_time", t0, t1)
            self.clock.span("backward_time", t1, self.clock.now())
        pool = self._pool
        pool.setdefault("loss", []).append(torch.stack([num.detach().float(), den.float()]))
        pool.setdefault("acc_pp", []).append(torch.stack([acc_pp * count_pp.clamp(min=1.0) * (count_pp > 0), count_pp]))
        pool.setdefault("loss_pp", []).append(torch.stack([loss_pp * count_pp.clamp(min=1.0) * (count_pp > 0), count_pp]))
        for key, value in comps.items():
            if key.startswith("_"):          # raw control statistics (e.g. Ling router counts): summed, not averaged
                pool.setdefault("x/" + key, []).append(value.float())
                continue
            n_, d_ = value
            pool.setdefault("c/" + key, []).append(torch.stack([n_.float().reshape(()), d_.float().reshape(())]))

    # -- one optimizer update -------------------------------------------------------------
    def train_update(self, batches: Iterable[dict]) -> None:
        """Run ``accumulation`` micro-batches and one optimizer step.  No host synchronisation."""
        self.model.train()
        self._pool = {}
        self.clock.reset()
        n = 0
        it = iter(batches)

        def fetch():
            h0 = time.perf_counter()
            staged = self._stage(next(it, None))
            self.clock.add_host("data_time", time.perf_counter() - h0)
            return staged

        staged = fetch()
        while staged is not None:
            batch, ready = staged
            staged = fetch()                              # the next micro-batch's copies run under this one's compute
            if ready is not None:
                torch.cuda.current_stream(self.device).wait_event(ready)
            self._forward_backward(batch)
            n += 1
        if n == 0:
            raise ValueError("train_update needs at least one micro-batch")
        opt = self.optimizer
        t_opt = self.clock.now()
        opt.fold_autograd_grads()
        pooled = {k: torch.stack(v).sum(0) for k, v in self._pool.items()}
        world = dist.get_world_size(self.dp_group) if (dist.is_available() and dist.is_initialized()) else 1
        if world > 1:
            keys = sorted(pooled)
            flat = torch.cat([pooled[k].reshape(-1) for k in keys])
            dist.all_reduce(flat, group=self.dp_group)
            off = 0
            for k in keys:
                m = pooled[k].numel()
                pooled[k] = flat[off:off + m].view_as(pooled[k])
                off += m
            if not self.sharded:            # the sharded optimizer reduces its own shard from the peers' buffers
                dense = getattr(opt, "dense_numel", opt.flat_grad.numel())
                dist.all_reduce(opt.flat_grad[:dense], group=self.dp_group)
                if dense < opt.flat_grad.numel() and self.expert_replica_group is not None:
                    # an expert's gradient already holds every token routed to it; only its replicas are summed
                    dist.all_reduce(opt.flat_grad[dense:], group=self.expert_replica_group)
        for hook in self.pre_step_hooks:     # debug dumps read the accumulated (not yet scaled) gradients here
            hook(self)
        den = pooled["loss"][1]
        opt.set_grad_scale(torch.where(den > 0, 1.0 / den.clamp(min=1e-12), torch.zeros_like(den)))
        grad_norm = opt.step()
        self.clock.span("optimizer_time", t_opt, self.clock.now())      # gradient reduction, clipping and the update
        self.global_step += 1
        counts = pooled.pop("x/_ling_router_counts", None)
        if counts is not None:
            self._update_router_bias(counts)
        for hook in self.post_step_hooks:
            hook(self)
        pooled["grad_norm"] = grad_norm
        self._last = pooled

    def _update_router_bias(self, counts: torch.Tensor) -> None:
        """Ling balancing: once per committed optimizer step, from the counts pooled over micro-batches and ranks
        (they were already SUM-reduced with the other pooled statistics)."""
        from aspec_b200.models.draft.ling_moe import LingMoE, update_ling_bias
        cfg = self.draft.config
        layers = [l.mlp for l in self.draft.layers if isinstance(getattr(l, "mlp", None), LingMoE)]
        if layers:
            update_ling_bias(layers, counts, cfg.moe_router_bias_update_rate, cfg.bias_zero_mean_update)

    # -- held-out evaluation: same forward and pooling as training, no gradients, no optimizer step ---------------
    # (reference: aspec/controller/eval.py:42-357, aspec/training/trainer.py:387-533)
    def eval_begin(self) -> dict:
        return {"pool": {}, "n": 0}

    @torch.no_grad()
    def eval_add(self, state: dict, batch: dict) -> None:
        was_training = self.model.training
        self.model.eval()
        saved = self._pool
        self._pool = state["pool"]
        try:
            self._forward_backward(self.to_device(batch))
            state["n"] += 1
        finally:
            self._pool = saved
            self.model.train(was_training)

    def eval_end(self, state: dict) -> Dict[str, float]:
        if state["n"] == 0:
            return {}
        pooled = {k: torch.stack(v).sum(0) for k, v in state["pool"].items()}
        world = dist.get_world_size(self.dp_group) if (dist.is_available() and dist.is_initialized()) else 1
        if world > 1:
            keys = sorted(pooled)
            flat = torch.cat([pooled[k].reshape(-1) for k in keys])
            dist.all_reduce(flat, group=self.dp_group)
            off = 0
            for k in keys:
                m = pooled[k].numel()
                pooled[k] = flat[off:off + m].view_as(pooled[k])
                off += m
        pooled["grad_norm"] = torch.zeros((), device=self.device)
        saved_last = self._last
        self._last = pooled
        try:
            out = {("eval/" + k[len("train/"):] if k.startswith("train/") else k): v for k, v in self.metrics().items()}
        finally:
            self._last = saved_last
        for drop in ("eval/grad_norm", "eval/lr", "eval/global_step"):
            out.pop(drop, None)
        return out

    def eval_update(self, batches: Iterable[dict]) -> Dict[str, float]:
        state = self.eval_begin()
        for b in batches:
            self.eval_add(state, b)
        return self.eval_end(state)

    def metrics(self) -> Dict[str, float]:
        """Metrics of the last update (one device->host transfer)."""
        p = self._last
        if not p:
            return {}
        keys = sorted(k for k in p if k != "grad_norm" and not k.startswith("x/"))
        flat = torch.cat([p[k].reshape(-1).float() for k in keys] + [p["grad_norm"].reshape(1).float()]).cpu()
        out: Dict[str, float] = {}
        off = 0
        vals = {}
        for k in keys:
            m = p[k].numel()
            vals[k] = flat[off:off + m].view_as(p[k].cpu())
            off += m
        out["train/grad_norm"] = float(flat[-1])
        phases = self.clock.totals()                     # the transfer above synchronised the stream: the events are done
        for name in ("data_time", "forward_time", "backward_time", "optimizer_time"):
            out["perf/" + name] = float(phases.get(name, 0.0))
        out["perf/compute_time"] = out["perf/forward_time"] + out["perf/backward_time"]
        num, den = vals["loss"]
        out["train/avg_loss"] = float(num / den) if den > 0 else 0.0
        a, c = vals["acc_pp"]
        out["train/avg_acc"] = float(a.sum() / c.sum()) if c.sum() > 0 else 0.0
        accs = (a / c.clamp(min=1.0)).tolist()
        tau, run = 0.0, 1.0
        for i, v in enumerate(accs):
            out[f"train/acc_{i}"] = v
            if c[i] > 0:
                run *= v
                tau += run
        out["train/simulated_acc_len"] = tau
        l_, c2 = vals["loss_pp"]
        for i, v in enumerate((l_ / c2.clamp(min=1.0)).tolist()):
            out[f"train/ploss_{i}"] = v
        for k in keys:
            if k.startswith("c/"):
                n_, d_ = vals[k]
                out["train/" + k[2:]] = float(n_ / d_) if d_ > 0 else 0.0
        out["train/lr"] = self.optimizer.get_learning_rate()
        out["train/global_step"] = self.global_step
        return out
