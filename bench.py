#!/usr/bin/env python
"""Headline benchmark: Draft input tokens/s of Qwen3-8B-shaped DSpark training at 4K.

``python bench.py --gpus N --steps K --warmup W`` (torchrun-launched for N > 1, one rank per GPU).

One *step* is one optimizer update over ``--accum`` documents per rank: forward, backward, gradient
reduction across ranks, clip, AdamW.  Documents follow the benchmark config: lengths log-uniform in
[256, 4096], uniform token ids, loss mask on the final 60 %, 512 anchors x block 7, one document per
micro-batch.  Features are synthetic (random bf16 captured layers) and weights random-init.

* ``value``: tokens/s with the documents' features resident on the GPU (the reference's Draft-only
  methodology), device-timed with CUDA events, max over ranks.  Anchors are sampled inside the timed region
  (on the host, from the host copy of the loss mask, as the data pipeline does).
* ``e2e.value``: the same metric through ``DraftTrainer.train_update`` fed from pinned host memory,
  every step including the host->device copy of its inputs and a device->host read of its metrics.
* for N >= 2 the gradient exchange and optimizer run over peer memory (sharded reduce + AdamW + parameter
  scatter kernels); ``--baseline`` keeps the NCCL all-reduce + replicated AdamW.
* for N >= 2 rank 0 afterwards runs the online split (N/2 Target + N/2 Draft GPUs, steady window of at least
  32 updates) as a child process and reports it under ``online``; ``--no-online`` skips it.
* ``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` and prints the same keys.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_1GPU = 15256.44   # published Draft-only tok/s, 1 x H200
BASELINE_8GPU = 77721.37   # published online tok/s, 8 x H200


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--accum", type=int, default=16, help="documents (micro-batches) per optimizer update per rank")
    ap.add_argument("--layers", type=int, default=1, help="Draft decoder layers (benchmark config: 1; reference recipe: 5)")
    ap.add_argument("--target-layers", type=int, default=3)
    ap.add_argument("--min-len", type=int, default=256)
    ap.add_argument("--max-len", type=int, default=4096)
    ap.add_argument("--pool", type=int, default=0, help="distinct documents per rank (0 = accum * 2)")
    ap.add_argument("--small", action="store_true", help="tiny shapes (CPU smoke / debugging only; not a valid bench)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mode", default="draft", choices=["draft", "online"],
                    help="draft: Draft-only data parallel (the `value`); online: Target + Draft ranks with feature rings")
    ap.add_argument("--targets", type=int, default=0, help="online: Target GPUs (default N // 2)")
    ap.add_argument("--target-layers-total", type=int, default=36)
    ap.add_argument("--target-batch", type=int, default=4, help="online: documents packed into one Target prefill")
    ap.add_argument("--length-group", type=int, default=32,
                    help="online: the controller's length_group_size (documents of similar length go to different Draft ranks "
                         "in the same micro-step; 1 disables the grouping)")
    ap.add_argument("--fsdp", action="store_true", help="draft mode, N >= 2: FULL_SHARD (parameters and gradients sharded per layer as well, gathered / reduce-scattered "
                         "over peer memory around every layer) instead of the default SHARD_OPTIMIZER step")
    ap.add_argument("--baseline", action="store_true",
                    help="draft mode, N >= 2: NCCL all-reduce of the flat gradient + replicated AdamW instead of the peer-memory sharded step")
    ap.add_argument("--no-online", action="store_true", help="N >= 2: do not append the online Target + Draft run")
    ap.add_argument("--online-steps", type=int, default=64, help="measured updates of the appended online run (window >= 32 updates)")
    ap.add_argument("--online-warmup", type=int, default=8)
    ap.add_argument("--online-timeout", type=float, default=900.0, help="seconds before the appended online run is abandoned")
    return ap.parse_args()


METRIC = "Draft input tokens/s, Qwen3-8B DSpark 4K (Draft-only, resident features)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._proc = index, [], False, None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()

    def _read(self):
        for line in self._proc.stdout:
            if self._stop:
                break
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        self._stop = True
        if self._proc is not None:
            self._proc.terminate()
        mhz, mx, reasons = [], 0, set()
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = max(mx, float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def build_ours(args, device, dtype):
    import torch
    from aspec_b200.config.draft_config import DSparkConfig
    from aspec_b200.models.draft.dspark import DSparkDraftModel
    from aspec_b200.models.dspark import DSparkModel
    if args.small:
        dims = dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1,
                    head_dim=128, vocab_size=4096, target_hidden_size=256, markov_rank=32, mask_token_id=4095)
    else:
        dims = dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
                    vocab_size=151936, target_hidden_size=4096, markov_rank=256, mask_token_id=151669)
    n_tl = args.target_layers
    ids = {3: [2, 18, 33], 5: [1, 9, 17, 25, 33]}.get(n_tl)
    cfg = DSparkConfig(num_hidden_layers=args.layers, num_target_layers=n_tl, target_layer_ids=ids,
                       target_num_hidden_layers=36, rope_theta=1e6, max_position_embeddings=40960, **dims)
    torch.manual_seed(1234)
    with torch.device(device):
        draft = DSparkDraftModel(cfg)
    draft = draft.to(dtype=dtype)
    model = DSparkModel(draft, block_size=7, num_anchors=512 if not args.small else 64,
                        loss_decay_gamma=4.0, ce_loss_alpha=0.1, l1_loss_alpha=0.9, confidence_head_alpha=1.0)
    lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, dtype=torch.float32) * 0.02).to(dtype)
    return cfg, model, lm_head


def make_pool(args, cfg, model, rank, n_docs, pin):
    """Host-side documents with features.  ``host_loss_mask`` stays on the host for the anchor sampler."""
    import torch
    from aspec_b200.data.synthetic import SyntheticSpec, benchmark_documents, synthetic_features
    spec = SyntheticSpec(vocab_size=cfg.vocab_size - 1024, min_len=min(args.min_len, args.max_len), max_len=args.max_len, seed=17)
    pool = []
    # every rank gets documents with the 1-GPU run's lengths (own token ids and features), dealt to the updates so that
    # each update carries about the same number of tokens: see ``benchmark_documents``
    for doc in benchmark_documents(spec, n_docs, args.accum, rank):
        row, T = doc["row"], doc["seq_len"]
        feats = synthetic_features(T, cfg.num_target_layers, cfg.target_hidden_size, row, pin=pin)
        lm = doc["loss_mask"][None]
        batch = {"input_ids": doc["input_ids"][None], "loss_mask": lm,
                 "hidden_states": feats["hidden_states"][None], "last_hidden_states": feats["last_hidden_states"][None],
                 "seq_len": T, "host_loss_mask": lm}
        if pin and torch.cuda.is_available():
            for k in ("input_ids", "loss_mask"):
                batch[k] = batch[k].pin_memory()
        pool.append(batch)
    return pool


def run_ours(args):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    if cuda:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", device_id=device if cuda else None)
    from aspec_b200 import _native
    from aspec_b200.ops.anchors import sample_anchor_positions
    from aspec_b200.training.draft_trainer import DraftTrainer
    cfg, model, lm_head = build_ours(args, device, dtype)
    total_updates = args.steps * 2 + args.warmup * 2 + 8
    sharded = world > 1 and not args.baseline
    trainer = DraftTrainer(model, lm_head, lr=6e-4, min_lr=6e-5, weight_decay=0.0, max_grad_norm=1.0,
                           total_steps=max(total_updates, 32), warmup_ratio=0.04, accumulation=args.accum,
                           device=device, fsdp_strategy=("FULL_SHARD" if args.fsdp else "SHARD_OPTIMIZER") if sharded else "REPLICATE")
    n_docs = args.pool or args.accum * 2
    pool = make_pool(args, cfg, model, rank, n_docs, pin=cuda)
    resident = [dict(trainer.to_device(b), host_loss_mask=b["host_loss_mask"]) for b in pool]
    if cuda:
        torch.cuda.synchronize()
    sampler_rng = torch.Generator().manual_seed(1000 + rank)

    def batches_for(step, source):
        """The step's micro-batches, each with anchors drawn now: the sampler's cost is inside the timed region."""
        out = []
        for i in range(args.accum):
            b = dict(source[(step * args.accum + i) % n_docs])
            lm = b.pop("host_loss_mask")
            anchors, keep = sample_anchor_positions(b["seq_len"], lm, model.num_anchors, model.block_size,
                                                    generator=sampler_rng)
            b["injected_anchors"], b["injected_keep_mask"] = anchors, keep
            out.append(b)
        return out

    def tokens_for(step):
        return sum(pool[(step * args.accum + i) % n_docs]["seq_len"] for i in range(args.accum))

    def barrier():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(source, read_metrics):
        for w in range(args.warmup):
            trainer.train_update(batches_for(w, source))
            if read_metrics:
                trainer.metrics()
        barrier()
        sampler = ClockSampler(local) if (cuda and rank == 0) else None
        if sampler:
            sampler.start()
        launches0 = _native.launch_count
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        toks = 0
        last = {}
        for s in range(args.steps):
            trainer.train_update(batches_for(args.warmup + s, source))
            toks += tokens_for(args.warmup + s)
            if read_metrics:
                last = trainer.metrics()
        if cuda:
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
        clocks = sampler.stop() if sampler else None
        launches = _native.launch_count - launches0
        stats = torch.tensor([ms, float(toks)], dtype=torch.float64, device=device)
        if world > 1:
            mx = stats.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = stats.clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            ms, toks = float(mx[0]), float(sm[1])
        return ms, toks, clocks, launches, last

    ms, toks, clocks, launches, _ = timed(resident, read_metrics=False)
    if cuda:
        from aspec_b200.ops.gemm import check_status
        check_status(device)
    value = toks / (ms / 1e3)
    e2e = None
    if not args.no_e2e:
        ms2, toks2, _, _, last = timed(pool, read_metrics=True)
        h2d = sum(DraftTrainer.h2d_bytes(b) for b in batches_for(args.warmup, pool))
        e2e = {"value": toks2 / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4 * (3 * 2 * model.block_size + 2 + 2 * 12 + 1),
               "ms_per_step": ms2 / args.steps, "loss": last.get("train/avg_loss")}
    collective = ("none (1 GPU)" if world == 1 else
                  "NCCL all-reduce of the flat fp32 gradient + replicated AdamW" if args.baseline else
                  "sharded step over gloo collectives (CPU run)" if not cuda else
                  "FULL_SHARD: per-layer peer_gather (peer loads) before forward and backward, per-layer shard_reduce_accum "
                  "(peer loads) under the backward of the layers below, flags in peer memory; NCCL only for the two-scalar "
                  "norm and the pooled metrics" if args.fsdp else
                  "peer-memory sharded step: shard_reduce_sumsq (peer loads) + shard_adamw_scatter (peer stores); "
                  "NCCL only for three scalar all-reduces per update")
    line = None
    if rank == 0:
        base = BASELINE_1GPU if world == 1 else None
        line = {
            "metric": METRIC,
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / base) if base else None, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (uniform token ids, log-uniform lengths, random bf16 features, random-init weights)",
            "config": {"model": f"Qwen3-8B-shaped DSpark draft, {args.layers} layer(s), {args.target_layers} captured layers, vocab {cfg.vocab_size}",
                       "global_batch": args.accum * world, "seq_len": args.max_len,
                       "doc_lengths": f"log-uniform [{args.min_len},{args.max_len}]",
                       "parallelism": f"dp{world}" + (("+full_shard" if args.fsdp else "+sharded_optimizer") if sharded else ""),
                       "collective": collective,
                       "anchors_sampled": "inside the timed region, every micro-batch",
                       "dp_balance": "every rank draws documents with the length sequence of the 1-GPU run (own token ids and features)" if world > 1 else "n/a", "micro_batch": "1 document (MBS1)", "anchors": model.num_anchors,
                       "block_size": model.block_size,
                       "l2_policy": "inputs larger than L2 (1.2 GB lm_head + per-document features stream from HBM every micro-batch)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "impl": "ours",
        }
    # release this rank's GPU before the online run takes the node
    close = getattr(trainer.optimizer, "close", None)
    if world > 1:
        dist.barrier()
    if close:
        close()
    del trainer, model, lm_head, resident, pool
    if cuda:
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        if world > 1 and cuda and not args.no_online and not args.small:
            line["online"] = online_with_split_search(args, draft_rate=value / world)
        print(json.dumps(line), flush=True)


def online_with_split_search(args, draft_rate: float) -> dict:
    """The online run at N/2 Target + N/2 Draft GPUs, then - when the measured service rates say another split is
    faster - at the split the topology search picks.  The better measured run is reported; both are listed under
    ``split_search`` so the choice can be checked."""
    from aspec_b200.topology import legal_splits, predict
    # a Draft rank fed over the feature rings trains at about 0.8 of its resident-feature rate (measured on B200s:
    # 78 K against 97.8 K tokens/s at 5 Target + 3 Draft GPUs); the rule is given that, not the resident rate
    ring_fed = 0.8
    first = online_child(args)
    tokens, busy = first.get("target_tokens") or [], first.get("target_busy_seconds") or []
    per_gpu = sorted(t / b for t, b in zip(tokens, busy) if t and b)
    search = {"draft_tokens_per_s_per_gpu": draft_rate, "ring_fed_draft_efficiency": ring_fed,
              "rule": "min(T x target rate, D x draft rate x ring-fed efficiency) over the legal splits",
              "runs": [{"split": f"{first.get('targets')}T+{first.get('drafts')}D", "value": first.get("value")}]}
    first["split_search"] = search
    if not per_gpu or not first.get("value"):
        return first
    target_rate = per_gpu[len(per_gpu) // 2]
    search["target_tokens_per_s_per_gpu"] = target_rate
    ranked = sorted(((predict(target_rate, draft_rate, t, d, ring_fed)[0], t, d) for t, d in legal_splits(args.gpus)), reverse=True)
    search["predicted"] = [{"split": f"{t}T+{d}D", "tokens_per_s": p} for p, t, d in ranked[:3]]
    best_p, best_t, best_d = ranked[0]
    here = predict(target_rate, draft_rate, first["targets"], first["drafts"], ring_fed)[0]
    if best_t == first["targets"] or best_p < 1.05 * here:
        return first
    second = online_child(args, targets=best_t)
    search["runs"].append({"split": f"{best_t}T+{best_d}D", "value": second.get("value"), "error": second.get("error")})
    if second.get("value") and second.get("ledger_validated") and second["value"] > first["value"]:
        second["split_search"] = search
        return second
    return first


def online_child(args, targets: int = 0) -> dict:
    """Run ``--mode online`` on the node's N GPUs in a child process (this process keeps only its CUDA context)."""
    time.sleep(3.0)                         # the other ranks are exiting and releasing their GPUs
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME",
                        "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_RESTART_COUNT",
                        "TORCHELASTIC_MAX_RESTARTS", "TORCHELASTIC_USE_AGENT_STORE", "TORCH_NCCL_ASYNC_ERROR_HANDLING",
                        "GROUP_WORLD_SIZE", "ROLE_WORLD_SIZE", "TORCHELASTIC_ERROR_FILE")}
    cmd = [sys.executable, os.path.abspath(__file__), "--mode", "online", "--gpus", str(args.gpus),
           "--steps", str(args.online_steps), "--warmup", str(args.online_warmup), "--accum", str(args.accum),
           "--layers", str(args.layers), "--min-len", str(args.min_len), "--max-len", str(args.max_len),
           "--targets", str(targets or args.targets or 0)]
    t0 = time.perf_counter()
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.online_timeout, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"error": f"online run did not finish within {args.online_timeout:.0f} s"}
    for ln in reversed(res.stdout.strip().splitlines()):
        if ln.startswith("{"):
            try:
                out = json.loads(ln)
                out["wall_seconds_incl_startup"] = time.perf_counter() - t0
                return out
            except json.JSONDecodeError:
                continue
    return {"error": f"online run exited {res.returncode}", "stderr_tail": res.stderr[-600:]}


def run_online(args) -> dict:
    """Online training on N GPUs of this node: T Target ranks prefill and store captured layers into the
    rings of D Draft ranks, which train.  Steady-window input tokens/s over committed work."""
    import tempfile

    import torch
    from aspec_b200.config.draft_config import DSparkConfig
    from aspec_b200.train_entry import train_async_no_generation
    n = args.gpus
    T = args.targets or max(n // 2, 1)
    D = n - T
    if D < 1:
        raise SystemExit("online mode needs at least one Draft GPU")
    small = args.small
    dims = (dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1, head_dim=128,
                 vocab_size=4096, target_hidden_size=256, markov_rank=32, mask_token_id=4095) if small else
            dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
                 vocab_size=151936, target_hidden_size=4096, markov_rank=256, mask_token_id=151669))
    L = 4 if small else args.target_layers_total
    ids = [0, 1, 3] if small else [2, 18, 33]
    draft = DSparkConfig(num_hidden_layers=args.layers, num_target_layers=3, target_layer_ids=ids,
                         target_num_hidden_layers=L, rope_theta=1e6, max_position_embeddings=40960, **dims).to_dict()
    steps = args.warmup + args.steps
    out_dir = tempfile.mkdtemp(prefix="aspec_online_")
    flat = dict(
        inference_engine_type="native", inference_num_gpus=T, training_num_gpus_per_node=D, training_num_nodes=1,
        world_size=D, draft_context_parallel_size=1, micro_batch_size=1, draft_accumulation_steps=args.accum,
        max_seq_length=args.max_len, num_train_steps=steps, learning_rate=6e-4, min_lr=6e-5, weight_decay=0.0,
        max_grad_norm=1.0, warmup_ratio=0.04, lr_decay_style="cosine", seed=0, dspark_block_size=7,
        dspark_num_anchors=64 if small else 512, dspark_loss_decay_gamma=4.0, dspark_ce_loss_alpha=0.1,
        dspark_l1_loss_alpha=0.9, dspark_confidence_head_alpha=1.0, train_data_path="synthetic",
        synthetic_num_documents=max(steps * args.accum * D * 2, 64), synthetic_min_length=min(args.min_len, args.max_len),
        synthetic_max_length=args.max_len, synthetic_vocab_size=dims["vocab_size"] - 1024, shuffle_dataset=True,
        length_group_size=max(args.length_group, 1), transport_destination_ring_slots=max(2 * args.accum + 2, 4),
        # batches are cut by tokens (about --target-batch average documents), so short documents still fill the GEMMs
        inference_batch_size=max(args.target_batch, 1) * 8, inference_batch_tokens=max(args.target_batch, 1) * 2048,
        store_last_hidden_states=True, output_dir=out_dir, save_interval=0, save_final_checkpoint=False,
        performance_warmup_steps=args.warmup, performance_drain_steps=0, optimizer_step_timeout_seconds=900.0,
        target_model_config={"model_type": "qwen3", "hidden_size": dims["hidden_size"], "intermediate_size": dims["intermediate_size"],
                             "num_hidden_layers": L, "num_attention_heads": dims["num_attention_heads"],
                             "num_key_value_heads": dims["num_key_value_heads"], "head_dim": 128,
                             "vocab_size": dims["vocab_size"], "rope_theta": 1e6},
        force_cpu=not torch.cuda.is_available(), num_epochs=1)
    summary = train_async_no_generation(flat, draft, log=lambda m: None)
    w = summary["window"]
    eng = summary.get("engines", [])
    steady = summary.get("history", [])[args.warmup:]
    med = lambda key: (sorted(h[key] for h in steady if key in h) or [None])[len([h for h in steady if key in h]) // 2]
    return {"value": w.get("tokens_per_second"), "unit": "tokens/s", "targets": T, "drafts": D,
            "steady_steps": w.get("steps"), "steady_tokens": w.get("tokens"), "steady_seconds": w.get("seconds"),
            "documents_per_update": args.accum * D, "ledger_validated": summary["ledger"]["validated"],
            # where an update's wall time goes: inside the trainer (waiting for rows + compute) and around it (driver)
            "median_trainer_step_seconds": med("perf/step_time"), "median_loop_step_seconds": med("perf/step_wall_time"),
            "vs_baseline_8gpu": (w.get("tokens_per_second") / BASELINE_8GPU) if (w.get("valid") and n == 8) else None,
            "target_busy_seconds": [e.get("busy_seconds") for e in eng], "target_tokens": [e.get("tokens") for e in eng],
            "timing": "steady window: from completion of warm-up update W to the last optimizer completion; each "
                      "completion is observed after a device-to-host read on every Draft rank"}


def run_reference(args):
    from baseline import reference_arm
    reference_arm.main(args)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    elif a.mode == "online":
        # one driver process owns the node: under torchrun only rank 0 drives, the other ranks just exit
        if int(os.environ.get("RANK", "0")) == 0:
            res = run_online(a)
            print(json.dumps({"metric": "online steady-window input tokens/s, Qwen3-8B DSpark 4K", "n_gpus": a.gpus,
                              "higher_is_better": True, "dtype": "bf16", "impl": "ours", **res}))
    else:
        run_ours(a)
