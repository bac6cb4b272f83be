"""One trainer process per Draft GPU.

Counterpart of the reference's Ray ``TrainerActor`` (aspec/training/trainer_actor.py:75-245): ``init``
joins the trainer process group, builds the Draft and its optimizer and allocates the feature ring that
Target ranks write into; ``train_from_queue(step, num_batches)`` pops sample descriptors, reads the
slots zero-copy, runs the micro-batches and the optimizer step, and reports metrics, the work it
consumed and the leases it no longer needs.
"""
from __future__ import annotations

import os
import queue as _queue
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from aspec_b200.config.draft_config import AutoDraftModelConfig
from aspec_b200.data.utils import unpack_loss_mask
from aspec_b200.training import checkpoint as ckpt
from aspec_b200.training.draft_trainer import DraftTrainer
from aspec_b200.training.factory import build_training_model
from aspec_b200.transport.feature_ring import FeatureDescriptor, FeatureRing, SlotLayout
from aspec_b200.utils.types import TrainSample


class TrainerActor:
    def __init__(self, rank: int, world: int, args: Dict[str, Any], draft_config: Dict[str, Any], train_queue,
                 master_port: int = 29517, group_name: str = "draft"):
        self.rank, self.world, self.args = rank, world, dict(args)
        self.queue = train_queue
        dev = self.args.get("trainer_devices", ["cpu"] * world)[rank]
        self.device = torch.device(dev)
        self.cuda = self.device.type == "cuda"
        if self.cuda:
            torch.cuda.set_device(self.device)
        self.dtype = torch.bfloat16 if self.cuda else torch.float32
        if world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ["MASTER_PORT"] = str(master_port)
            # a collective that a lost rank never joins ends with an error after this long instead of waiting forever
            from datetime import timedelta
            dist.init_process_group("nccl" if self.cuda else "gloo", rank=rank, world_size=world,
                                    device_id=self.device if self.cuda else None,
                                    timeout=timedelta(minutes=float(self.args.get("distributed_timeout_minutes") or 10)))
        torch.manual_seed(int(self.args.get("seed", 0)))
        # nothing in training draws from these two, but they are part of the checkpointed RNG state: seeded, two runs of
        # one recipe write identical checkpoints
        import random
        random.seed(int(self.args.get("seed", 0)) * 1000003 + rank)
        try:
            import numpy as np
            np.random.seed((int(self.args.get("seed", 0)) * 1000003 + rank) % (2 ** 32))
        except ImportError:          # pragma: no cover
            pass
        self.draft_config = AutoDraftModelConfig.from_dict(draft_config)
        self.model = build_training_model(self.draft_config, self.args, self.device, self.dtype)
        self._load_native_mtp()                  # before the optimizer takes its fp32 masters from the weights
        if self.args.get("initial_draft_model_path") and not self.args.get("load_path"):
            self._load_initial_weights(str(self.args["initial_draft_model_path"]))
        cfg = self.draft_config
        self.expert_parallel = None
        ep = max(int(self.args.get("expert_parallel_size", 1) or 1), 1)
        if ep > 1:
            # ranks [g * ep, (g + 1) * ep) hold all experts between them; ranks r, r + ep, ... hold replicas
            if world < ep or world % ep:
                raise ValueError("expert_parallel_size must divide the Draft world size")
            if str(self.args.get("fsdp_strategy", "REPLICATE")).upper() == "FULL_SHARD":
                raise ValueError("expert parallelism shards the experts itself; use fsdp_strategy=REPLICATE with it")
            from aspec_b200.parallel.expert_wiring import apply_expert_parallel, attach_fused_exchange, build_groups
            group, replicas = build_groups(rank, world, ep)
            self.expert_parallel = apply_expert_parallel(self.model.draft_model, rank % ep, ep, group, replicas)
            if self.cuda:
                top_k = int(getattr(cfg, "num_experts_per_tok", 1) or 1)
                rows = (int(getattr(self.model, "num_anchors", 0) or 0) * int(getattr(self.model, "block_size", 1) or 1)
                        or int(self.args["max_seq_length"])) * top_k
                attach_fused_exchange(self.expert_parallel, rows, int(cfg.hidden_size), self.device)
        self.cp_size = max(int(self.args.get("draft_context_parallel_size", 1) or 1), 1)
        if self.cp_size > 1 and hasattr(self.model, "context_parallel") and world > 1:
            # ranks [g * cp, (g + 1) * cp) share every row: each projects its context shard and carries its own blocks
            from aspec_b200.parallel.cp_runtime import ContextParallel, attach
            if world % self.cp_size:
                raise ValueError("draft_context_parallel_size must divide the Draft world size")
            groups = [dist.new_group(list(range(g * self.cp_size, (g + 1) * self.cp_size))) for g in range(world // self.cp_size)]
            per_rank = -(-int(self.model.num_anchors) // self.cp_size) * int(self.model.block_size)
            attach(self.model, ContextParallel(groups[rank // self.cp_size], num_layers=int(cfg.num_hidden_layers),
                                               max_queries=per_rank, heads=int(cfg.num_attention_heads),
                                               head_dim=int(cfg.head_dim), device=self.device))
        # a sequence-parallel group of ``u * r`` ranks shares every row: ``u`` adjacent ranks exchange heads (Ulysses), the
        # ``r`` blocks of ``u`` ranks pass key / value shards around a ring (reference: aspec/utils/distributed.py:117-201)
        self.sp_ulysses = max(int(self.args.get("sp_ulysses_size", 1) or 1), 1)
        self.sp_ring = max(int(self.args.get("sp_ring_size", 1) or 1), 1)
        self.sp_size = self.sp_ulysses * self.sp_ring
        if self.sp_size > 1 and world > 1 and getattr(self.model, "supports_sequence_parallel", False):
            # ranks [g * sp, (g + 1) * sp) share every row: each keeps a slice of the tokens
            u, r = self.sp_ulysses, self.sp_ring
            if world % self.sp_size:
                raise ValueError("sp_ulysses_size * sp_ring_size must divide the Draft world size")
            heads, kv_heads, hd = int(cfg.num_attention_heads), int(cfg.num_key_value_heads), int(cfg.head_dim)
            if heads % u or kv_heads % u:
                raise ValueError("sp_ulysses_size must divide the attention head counts")
            # every rank creates every group, in the same order
            sp_groups = [dist.new_group(list(range(g * self.sp_size, (g + 1) * self.sp_size))) for g in range(world // self.sp_size)]
            u_groups, ring_groups = {}, {}
            for g in range(world // self.sp_size):
                base = g * self.sp_size
                for b in range(r):
                    u_groups[(g, b)] = dist.new_group([base + b * u + i for i in range(u)]) if u > 1 else None
                for i in range(u):
                    ring_groups[(g, i)] = dist.new_group([base + b * u + i for b in range(r)]) if r > 1 else None
            g, idx = rank // self.sp_size, rank % self.sp_size
            mine = sp_groups[g]
            u_group, ring_group = u_groups[(g, idx // u)], ring_groups[(g, idx % u)]
            if self.cuda:
                from aspec_b200.parallel.group import exchange_workspaces, make_barrier
                from aspec_b200.parallel.ulysses import UlyssesExchange, UlyssesWorkspace
                rows = -(-int(self.args["max_seq_length"]) // self.sp_size) + 8
                own = UlyssesWorkspace(u, rows, (heads + 2 * kv_heads) * hd // u, heads * hd // u, device=self.device)
                if u > 1:
                    ws = exchange_workspaces(own, UlyssesWorkspace.open, group=u_group)
                    exchange = UlyssesExchange(idx % u, u, ws, make_barrier(self.device, u_group))
                else:                            # ring only: the projections run through the same kernels, no peers
                    exchange = UlyssesExchange(0, 1, [own], lambda: None)
            else:
                from aspec_b200.parallel.ulysses import CollectiveUlyssesExchange
                exchange = CollectiveUlyssesExchange(idx % u, u, u_group)
            self.model.draft_model.ulysses = exchange
            if r > 1:
                self.model.draft_model.ring = (idx // u, r, ring_group)
            self.model.sequence_parallel = (idx, self.sp_size, mine)
        # a row holds one packed row of at most ``max_seq_length`` tokens, or ``micro_batch_size`` whole documents
        row_tokens = int(self.args["max_seq_length"]) * (1 if self.args.get("dflash_packing") else max(int(self.args.get("micro_batch_size", 1)), 1))
        layout = SlotLayout(row_tokens, int(getattr(cfg, "num_target_layers", None)
                                                                   or getattr(cfg, "num_aux_hidden_states", 3)),
                            int(getattr(cfg, "target_hidden_size", cfg.hidden_size)),
                            bool(self.args.get("store_last_hidden_states", True)),
                            "bfloat16" if self.cuda else "float32")
        self.ring = FeatureRing(int(self.args.get("transport_destination_ring_slots", 4)), layout, self.device,
                                run_id=str(self.args.get("run_id", "run")), attempt_id=str(self.args.get("attempt_id", "0")),
                                consumer=int(self.args.get("consumer_base", 0)) + rank)
        self.trainer: Optional[DraftTrainer] = None
        self.fault: Optional[dict] = self.args.get("fault_injection")      # host-side: {"kind": "raise"|"sleep", "step": k}
        self._pending_releases: List[tuple] = []
        self._debug_instruments()

    @torch.no_grad()
    def _load_native_mtp(self) -> None:
        """Native MTP predictors start from (native-MTP training) or stay frozen at (MTP-conditioned blocks) the ``mtp.*``
        tensors of the Target checkpoint: ``model.mtp_source_path``, else ``model.target_model_path`` when that is a
        checkpoint directory that holds them.  A resume or an initial Draft asset loaded afterwards takes precedence for
        trainable tensors."""
        draft = self.model.draft_model
        if getattr(draft, "mtp_source", None) is not None:
            load = draft.initialize_mtp_conditioning
        elif type(draft).__name__ == "NativeMTPDraftModel":
            load = draft.initialize_native_weights
        else:
            return
        explicit = self.args.get("mtp_source_path")
        source = explicit or self.args.get("target_model_path")
        if not source or not os.path.isdir(str(source)):
            if explicit:
                raise FileNotFoundError(f"model.mtp_source_path {explicit} is not a checkpoint directory")
            return
        from aspec_b200.models.dmtp import read_native_mtp_tensors
        tensors = read_native_mtp_tensors(str(source))
        if not tensors:
            if explicit:
                raise ValueError(f"{explicit} holds no mtp.* tensors")
            return
        load({k: v.to(self.device) for k, v in tensors.items()})

    @torch.no_grad()
    def _load_initial_weights(self, asset_dir: str) -> None:
        """Start from an exported Draft (``model.initial_draft_model_path``): its tensors are copied into the freshly
        built modules in place, before the optimizer takes its fp32 masters from them.  The asset must hold exactly
        this architecture's tensors; a resume (``load_path``) takes precedence over it
        (reference: aspec/training/checkpoint.py:772-858)."""
        from safetensors.torch import load_file
        from aspec_b200.draft_artifact import validate_native_asset
        validate_native_asset(asset_dir)
        tensors = load_file(os.path.join(asset_dir, "model.safetensors"))
        draft = self.model.draft_model
        own = draft.state_dict()
        wrong = sorted(k for k in tensors if k in own and tuple(tensors[k].shape) != tuple(own[k].shape))
        if set(tensors) != set(own) or wrong:
            missing, extra = sorted(set(own) - set(tensors)), sorted(set(tensors) - set(own))
            raise ValueError(f"initial Draft asset {asset_dir} does not fit this Draft configuration: missing {missing[:4]}, "
                             f"unexpected {extra[:4]}, shape mismatch {wrong[:4]}")
        draft.load_state_dict({k: v.to(self.device) for k, v in tensors.items()}, strict=True)

    def _debug_instruments(self) -> None:
        """Profiler window, memory snapshot, step dumps and the JSONL timeline, all off unless the ``debug`` /
        ``logging`` sections ask for them.  Their files go under the run directory (``traces/``, ``dumps/``,
        ``timeline/``) unless a directory is configured."""
        from aspec_b200.utils.profiling import StepProfiler
        from aspec_b200.utils.timeline import Timeline
        a, out = self.args, str(self.args.get("output_dir") or ".")
        start, end = int(a.get("profile_step_start") or 0), int(a.get("profile_step_end") or 0)
        window = bool(a.get("use_pytorch_profiler")) and end > start
        mem_step = a.get("memory_snapshot_num_steps") if a.get("record_memory_history") else None
        trace_dir = a.get("profile_dir_name") if a.get("profile_dir_name") not in (None, "", "/tmp/aspec_profiles") else os.path.join(out, "traces")
        self.profiler = (StepProfiler(trace_dir, start if window else None, end if window else None,
                                      int(mem_step) if mem_step is not None else None, rank=self.rank)
                         if window or mem_step is not None else None)
        self.dump_dir = a.get("save_debug_train_data")
        if self.dump_dir in (True, "true", "1"):
            self.dump_dir = out
        self.timeline = Timeline((a.get("timeline_output_dir") or os.path.join(out, "timeline")) if a.get("timeline_enabled") else None,
                                 role="trainer", rank=self.rank, run_id=str(a.get("timeline_run_id") or a.get("run_id", "")),
                                 flush_every=int(a.get("timeline_flush_every") or 128), enabled=bool(a.get("timeline_enabled")))

    def observed_capabilities(self) -> dict:
        """Counts of the implementations that this process really ran, per subsystem."""
        from aspec_b200.ops.observed import snapshot
        return snapshot()

    # -- setup ------------------------------------------------------------------------------------
    def ring_handle(self, copies: int = 1) -> list:
        """One handle per producer process that will map this ring."""
        return [self.ring.export() for _ in range(max(int(copies), 1))]

    def set_vocab_mapping(self, d2t: torch.Tensor, t2d: torch.Tensor) -> None:
        """Draft vocabulary of a pruned output head: which Target tokens it predicts (reference:
        aspec/training/eagle3_trainer.py, ``vocab_mapping_path``).  A checkpoint loaded afterwards overrides it."""
        draft = self.model.draft_model
        if not getattr(draft, "vocab_pruned", False):
            raise ValueError("this Draft predicts the whole Target vocabulary")
        draft.set_vocab_buffers(d2t.to(draft.d2t.device), t2d.to(draft.t2d.device))

    def set_head(self, lm_head: Optional[torch.Tensor], embedding: Optional[torch.Tensor] = None) -> None:
        """Frozen Target output head (and embedding): a tensor, a relayable handle, ``{"file": path}`` (a head stored
        beside offline features) or ``None`` -> deterministic random init (feature stores without a head)."""
        from aspec_b200.transport.feature_ring import import_tensor
        cfg = self.draft_config
        if isinstance(lm_head, dict) and "file" in lm_head:
            lm_head = torch.load(lm_head["file"], map_location="cpu")
            if tuple(lm_head.shape) != (cfg.vocab_size, getattr(cfg, "target_hidden_size", None) or cfg.hidden_size):
                raise ValueError(f"stored Target head {tuple(lm_head.shape)} does not fit the Draft configuration")
        elif isinstance(lm_head, dict):
            lm_head = import_tensor(lm_head)
        if isinstance(embedding, dict) and "file" in embedding:
            embedding = torch.load(embedding["file"], map_location="cpu")
        elif isinstance(embedding, dict):
            embedding = import_tensor(embedding)
        if lm_head is None:
            g = torch.Generator().manual_seed(1234)
            lm_head = torch.randn(cfg.vocab_size, cfg.hidden_size, generator=g) * 0.02
        self.lm_head = lm_head.to(self.device, self.dtype).clone()     # own copy: the Target may live elsewhere
        vp = int(self.args.get("vocab_parallel_size", 1) or 1)
        if vp > 1 and self.cuda and hasattr(self.model, "prediction_start"):
            # ranks [g * vp, (g + 1) * vp) train on the same rows; each keeps 1 / vp of the head's rows
            from aspec_b200.parallel.group import exchange_workspaces, make_barrier
            from aspec_b200.parallel.vocab_parallel import VocabParallelHead, VocabShardWorkspace
            if self.world % vp:
                raise ValueError("vocab_parallel_size must divide the Draft world size")
            ranks = [list(range(g * vp, (g + 1) * vp)) for g in range(self.world // vp)]
            groups = [dist.new_group(r) for r in ranks]
            mine = groups[self.rank // vp]
            rows = int(self.args.get("dspark_num_anchors", self.args.get("dflash_num_anchors", 512))) * int(self.model.block_size)
            ws = exchange_workspaces(VocabShardWorkspace(rows, int(self.args["max_seq_length"]) + int(self.model.block_size) + 2,
                                                         cfg.hidden_size, int(getattr(cfg, "markov_rank", 0) or 8), vp,
                                                         device=self.device), VocabShardWorkspace.open, group=mine)
            head = VocabParallelHead(self.rank % vp, vp, cfg.vocab_size, ws, make_barrier(self.device, mine))
            self.model.vocab_parallel = head
            self.lm_head = head.shard_rows(self.lm_head).contiguous()
        draft = self.model.draft_model
        if embedding is not None and hasattr(draft, "load_embedding"):
            draft.load_embedding(embedding.to(self.device))
        a = self.args
        total = int(a.get("lr_total_steps") or a.get("num_train_steps") or 1000)
        wsd = {}
        if a.get("lr_decay_style") == "WSD":     # warm-up, stable, then a final decay over ``ratio`` of the schedule
            ratio = float(a.get("wsd_decay_ratio") if a.get("wsd_decay_ratio") is not None else a.get("lr_wsd_decay_ratio", 0.2))
            wsd = {"wsd_decay_steps": min(max(int(round(total * ratio)), 1), total),
                   "wsd_decay_style": a.get("wsd_decay_style") or a.get("lr_wsd_decay_style") or "cosine"}
        self.trainer = DraftTrainer(self.model, self.lm_head, lr=a.get("learning_rate", 1e-4), min_lr=a.get("min_lr", 0.0),
                                    weight_decay=a.get("weight_decay", 0.0), max_grad_norm=a.get("max_grad_norm", 0.5),
                                    total_steps=total, **wsd,
                                    warmup_ratio=a.get("warmup_ratio", 0.015), decay_style=a.get("lr_decay_style", "cosine"),
                                    accumulation=int(a.get("draft_accumulation_steps", 1)), device=self.device,
                                    fsdp_strategy=str(a.get("fsdp_strategy", "REPLICATE")))
        if self.expert_parallel is not None:
            plan = self.expert_parallel
            self.trainer.optimizer.set_expert_parallel(plan.group, plan.ep_rank, plan.ep_size)
            self.trainer.expert_replica_group = plan.replica_group

    # -- data ---------------------------------------------------------------------------------------
    def _batch(self, sample: TrainSample) -> dict:
        views = self.ring.read(sample.feature_key, device_flags=bool(self.args.get("device_flags", False)),
                               wait_limit_ms=float(self.args.get("transport_device_wait_limit_ms", 2000.0)))
        lens = tuple(sample.document_lengths)
        T = sum(lens)
        masks = [unpack_loss_mask(m, n) for m, n in zip(sample.packed_loss_masks, lens)]
        loss_mask = torch.cat(masks)[None]
        batch = {"input_ids": views["input_ids"][None], "hidden_states": views["hidden_states"][None],
                 "loss_mask": loss_mask, "_work": sample.metadata, "_aspec_work": sample.metadata,
                 "_key": sample.feature_key}
        if "last_hidden_states" in views:
            batch["last_hidden_states"] = views["last_hidden_states"][None]
        ctx_docs = None
        if len(lens) > 1:
            ctx_docs = torch.cat([torch.full((n,), i, dtype=torch.long) for i, n in enumerate(lens)])[None]
            batch["ctx_doc_ids"] = ctx_docs
            batch["base_position_ids"] = torch.cat([torch.arange(n) for n in lens])[None]
            batch["packed_document_lengths"] = lens
        if hasattr(self.model, "sample_anchors"):
            seed = None
            if getattr(self, "cp_size", 1) > 1 or self.args.get("deterministic_anchor_sampling"):
                # every rank of a context-parallel group must draw the same anchors for the row; with
                # ``deterministic_anchor_sampling`` the draw depends on the row alone, so that the same recipe trains
                # on the same blocks under any parallel layout
                import zlib
                # (by the documents it holds, not by its number: row numbers depend on how updates are dealt to ranks)
                seed = zlib.crc32("|".join(str(d) for d in sample.data_ids).encode()) ^ int(self.args.get("seed", 0))
            anchors, keep = self.model.sample_anchors(loss_mask, ctx_docs, lens if len(lens) > 1 else None, anchor_seed=seed)
            batch["injected_anchors"], batch["injected_keep_mask"] = anchors, keep
        return batch

    def _samples(self, num_batches: int, timeout: float, evaluation: bool = False):
        """Training and held-out samples share the queue (rows whose id starts with ``eval-`` are held-out); a sample
        of the other kind that arrives first is set aside and served to the next reader of its kind."""
        deadline = time.monotonic() + timeout
        stash = self.__dict__.setdefault("_stash", [])
        for _ in range(num_batches):
            item = None
            for i, held in enumerate(stash):
                if str(held.row_id).startswith("eval-") == evaluation:
                    item = stash.pop(i)
                    break
            while item is None:
                try:
                    got = self.queue.get(timeout=0.2)
                except _queue.Empty:
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"trainer {self.rank}: no sample within {timeout}s") from None
                    continue
                if got is None:
                    raise RuntimeError("train queue was closed")
                if str(got.row_id).startswith("eval-") == evaluation:
                    item = got
                else:
                    stash.append(got)
            yield item

    # -- the step ---------------------------------------------------------------------------------
    def train_from_queue(self, step: int, num_batches: int, timeout: float = 1800.0) -> dict:
        if self.fault and int(self.fault.get("step", -1)) == step and int(self.fault.get("rank", 0)) == self.rank:
            if self.fault.get("kind") == "sleep":
                time.sleep(float(self.fault.get("seconds", 3600)))
            elif self.fault.get("kind") == "exit":          # the process disappears between two updates (a lost node)
                os._exit(int(self.fault.get("code", 17)))
            else:
                raise RuntimeError(f"trainer {self.rank}: injected failure at step {step}")
        consumed, keys = [], []
        t0 = time.perf_counter()

        dumping = bool(self.dump_dir) and step < int(self.args.get("max_dump_steps") or 0)
        first_batch: dict = {}

        def batches():
            for sample in self._samples(num_batches, timeout):
                with self.timeline.span("batch_ready", step=step, rows=len(sample.metadata)):
                    b = self._batch(sample)
                if dumping and not first_batch:
                    first_batch.update(b)
                consumed.extend(m["execution_id"] for m in sample.metadata)
                keys.append(sample.feature_key)
                yield b

        grad_norms: dict = {}

        def capture_grad_norms(trainer) -> None:          # accumulated over the update, before the 1 / denominator scale
            for name, p in trainer.draft.named_parameters():
                g = getattr(p, "main_grad", None)
                g = p.grad if g is None else g
                if g is not None:
                    grad_norms[name] = float(g.float().norm())

        if self.profiler is not None:
            self.profiler.step(step)
        if dumping:
            self.trainer.pre_step_hooks.append(capture_grad_norms)
        try:
            with self.timeline.span("train_update", step=step, micro_batches=num_batches):
                self.trainer.train_update(batches())
                metrics = self.trainer.metrics()      # one device->host read; also orders the slot reuse
        finally:
            if dumping:
                self.trainer.pre_step_hooks.remove(capture_grad_norms)
        if dumping:
            from aspec_b200.utils.train_dump import dump_step
            dump_step(str(self.dump_dir), step, self.rank, batch=first_batch, outputs=dict(metrics), model=self.model,
                      grad_norms=grad_norms)
        if self.cuda:
            self.ring.check_status()
            from aspec_b200.ops.gemm import check_status
            check_status(self.device)
        releases = []
        for k in keys:
            d = FeatureDescriptor.from_key(k)
            releases.append((d.consumer, d.slot, d.generation))
        metrics["perf/step_time"] = time.perf_counter() - t0
        return {"metrics": metrics, "committed": consumed, "releases": releases, "step": step}

    # -- evaluation -------------------------------------------------------------------------------
    def eval_begin(self, cache_key: str = "") -> None:
        self._eval = {"key": cache_key, "kept": [], "state": self.trainer.eval_begin()}

    def eval_step(self, num_batches: int, timeout: float = 1800.0) -> dict:
        """Held-out forward over ``num_batches`` ring samples; the leases are returned at once so that a small ring
        suffices.  With a cache key the batches are kept in host memory for later passes."""
        keys = []
        ev = self._eval
        for sample in self._samples(num_batches, timeout, evaluation=True):
            b = self._batch(sample)
            keys.append(sample.feature_key)
            if ev["key"]:
                ev["kept"].append({k: (v.detach().to("cpu", copy=True) if torch.is_tensor(v) else v) for k, v in b.items()})
            self.trainer.eval_add(ev["state"], b)
        if self.cuda:
            torch.cuda.synchronize(self.device)            # the slots are reusable once the forward has read them
        releases = []
        for k in keys:
            d = FeatureDescriptor.from_key(k)
            releases.append((d.consumer, d.slot, d.generation))
        return {"releases": releases}

    def eval_end(self) -> dict:
        ev = self._eval
        metrics = self.trainer.eval_end(ev["state"])
        if ev["key"]:
            self._eval_cache = {"key": ev["key"], "batches": ev["kept"]}
        self._eval = None
        return {"metrics": metrics, "cached": len(ev["kept"])}

    def eval_from_cache(self, cache_key: str) -> dict:
        cache = getattr(self, "_eval_cache", None)
        if not cache or cache["key"] != cache_key:
            return {"metrics": {}, "miss": True}
        state = self.trainer.eval_begin()
        for b in cache["batches"]:
            self.trainer.eval_add(state, b)
        return {"metrics": self.trainer.eval_end(state), "miss": False}

    def decode_from_cache(self, cache_key: str, anchors_per_doc: int = 8, max_docs: int = 64) -> dict:
        """Train-with-decode: block proposals of the live Draft weights (no export, no reload) on the cached held-out
        rows, verified greedily against each document's continuation - mean accepted length tau during training
        (the reference drives a serving engine's speculative decode from the trainer for the same number,
        aspec/inference/engine/sgl_engine_decode.py:39-424)."""
        cache = getattr(self, "_eval_cache", None)
        if not cache or cache["key"] != cache_key:
            return {"miss": True}
        from aspec_b200.commands.evaluate_draft import evaluate
        from aspec_b200.draft_artifact import BlockDraftConsumer
        draft = self.model.draft_model
        was_training = draft.training
        if getattr(self.model, "vocab_parallel", None) is not None:
            return {"unsupported": "the output head is sharded over a vocabulary-parallel group"}
        try:
            consumer = BlockDraftConsumer(draft, block_size=int(self.model.block_size))
        except ValueError as exc:
            return {"unsupported": str(exc)}
        docs = []
        for b in cache["batches"]:
            ids, feats = b["input_ids"][0], b["hidden_states"][0]
            lens = b.get("packed_document_lengths") or (ids.numel(),)
            off = 0
            for n in lens:
                docs.append({"input_ids": ids[off:off + n], "features": feats[off:off + n]})
                off += n
        docs = docs[:max_docs]
        dtype = next(draft.parameters()).dtype
        try:
            res = evaluate(consumer, self.lm_head, docs,
                           lambda d: d["features"][None].to(self.device, dtype), anchors_per_doc=anchors_per_doc,
                           seed=int(self.args.get("seed", 0)))
        finally:
            draft.train(was_training)
        return {"decode": res, "miss": False}

    # -- checkpoints --------------------------------------------------------------------------------
    def topology(self) -> dict:
        return ckpt.logical_training_topology({**self.args, "world_size": self.world}, self.draft_config)

    def save_model(self, output_dir: str, step_id: int) -> str:
        return ckpt.save(output_dir=output_dir, step_id=step_id, model=self.model.draft_model,
                         optimizer=self.trainer.optimizer, draft_config=self.draft_config, topology=self.topology(),
                         global_step=self.trainer.global_step)

    def export_draft_asset(self, output_dir: str) -> Optional[dict]:
        """The live Draft weights as a native asset for the decoding Target engines.  Every rank joins (sharded
        parameters are gathered); rank 0 writes."""
        from aspec_b200.draft_artifact import write_live_asset
        with ckpt.whole_parameters(self.trainer.optimizer):
            if self.rank != 0:
                return None
            return write_live_asset(self.model.draft_model, output_dir, block_size=getattr(self.model, "block_size", None),
                                    source=f"update {self.trainer.global_step}")

    def load_model(self, load_path: str, continual: bool = False) -> dict:
        info = ckpt.load(load_path=load_path, model=self.model.draft_model, optimizer=self.trainer.optimizer,
                         topology=self.topology(), continual_training=continual)
        self.trainer.global_step = info["global_step"]
        if not continual:
            ckpt.finalize_load(info["checkpoint_dir"])
        return {k: info[k] for k in ("next_step", "global_step", "work_state", "checkpoint_dir")}

    def flush_debug(self) -> list:
        """Finish an open profiler window and flush the timeline; returns the trace files written so far."""
        if self.profiler is not None:
            self.profiler.close()
        self.timeline.close()
        return list(self.profiler.written) if self.profiler is not None else []

    def close(self) -> None:
        self.flush_debug()
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
