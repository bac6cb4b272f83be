"""Reference arm of the benchmark: the unmodified reference package (installed under ``baseline/_ref``) runs the
same Draft-only workload through its own public API - ``AutoDraftModelConfig`` / ``AutoEagle3DraftModel`` /
``DSparkModel`` / ``BF16Optimizer`` (aspec/models/dspark.py:71, aspec/training/optimizer.py:40) - with its stock
attention backend.  Nothing from ``aspec_b200`` is on the timed path; only the synthetic documents are shared so
that both arms see identical shapes.

The reference's numerator/denominator normalisation of an accumulation window
(aspec/training/dflash_trainer.py:489-533) is restated in the loop: ``backward(numerator / accumulation)`` per
micro-batch, then every gradient is scaled by ``accumulation / sum(denominators)`` before the optimizer step.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _unavailable(reason: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")[:300]}))


def main(args) -> None:
    try:
        result = _run(args)
    except Exception as exc:  # the contract: say why and exit 0
        _unavailable(f"{type(exc).__name__}: {exc}")
        return
    if result is not None:
        print(json.dumps(result))


def _run(args):
    import torch
    import torch.distributed as dist

    ref = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref, "aspec")):
        raise RuntimeError("baseline/_ref is absent (offline install not present)")
    sys.path.insert(0, ref)
    try:
        import omegaconf  # noqa: F401
    except ImportError:
        sys.path.insert(0, os.path.join(HERE, "shims"))
    from aspec.models.draft.dspark import DSparkConfig, DSparkDraftModel
    from aspec.models.dspark import DSparkModel
    from aspec.training.optimizer import BF16Optimizer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo")
    dtype = torch.bfloat16 if cuda else torch.float32

    if args.small:
        dims = dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1,
                    head_dim=128, vocab_size=4096, target_hidden_size=256, markov_rank=32, mask_token_id=4095)
    else:
        dims = dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
                    head_dim=128, vocab_size=151936, target_hidden_size=4096, markov_rank=256, mask_token_id=151669)
    n_tl = args.target_layers
    ids = {3: [2, 18, 33], 5: [1, 9, 17, 25, 33]}.get(n_tl)
    cfg = DSparkConfig(num_hidden_layers=args.layers, num_target_layers=n_tl, target_layer_ids=ids,
                       target_num_hidden_layers=36, rope_theta=1e6, max_position_embeddings=40960,
                       rms_norm_eps=1e-6, **dims)
    torch.manual_seed(1234)
    draft = DSparkDraftModel(cfg).to(device=device, dtype=dtype)
    backend = os.environ.get("ASPEC_REFERENCE_ATTENTION_BACKEND", "flex_attention")
    model = DSparkModel(draft, block_size=7, num_anchors=512 if not args.small else 64, loss_decay_gamma=4.0,
                        ce_loss_alpha=0.1, l1_loss_alpha=0.9, confidence_head_alpha=1.0, attention_backend=backend)
    model.train()
    lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, dtype=torch.float32) * 0.02).to(dtype)
    opt = BF16Optimizer(draft, lr=1e-4, weight_decay=0.0, max_grad_norm=0.5, total_steps=100000) if cuda else None
    params = [p for p in draft.parameters() if p.requires_grad]

    # same synthetic documents as the other arm (host tensors only; no model / kernel code is shared)
    sys.path.insert(0, os.path.dirname(HERE))
    from aspec_b200.data.synthetic import SyntheticSpec, benchmark_documents, synthetic_features
    spec = SyntheticSpec(vocab_size=cfg.vocab_size - 1024, min_len=min(args.min_len, args.max_len),
                         max_len=args.max_len, seed=17)
    n_docs = args.pool or args.accum * 2
    pool = []
    for doc in benchmark_documents(spec, n_docs, args.accum, rank):
        feats = synthetic_features(doc["seq_len"], n_tl, cfg.target_hidden_size, doc["row"], pin=cuda)
        pool.append({"input_ids": doc["input_ids"][None], "loss_mask": doc["loss_mask"][None],
                     "hidden_states": feats["hidden_states"][None], "last_hidden_states": feats["last_hidden_states"][None],
                     "seq_len": doc["seq_len"]})

    def update(step: int) -> int:
        tokens = 0
        dens = []
        for m in range(args.accum):
            b = pool[(step * args.accum + m) % n_docs]
            dev = {k: v.to(device, non_blocking=True) for k, v in b.items() if torch.is_tensor(v)}
            out = model(dev["input_ids"], dev["hidden_states"].to(dtype), dev["loss_mask"], lm_head,
                        last_hidden_states=dev["last_hidden_states"].to(dtype))
            num, den = out[6]
            (num / args.accum).backward()
            dens.append(den.detach().float())
            tokens += b["seq_len"]
        den = torch.stack(dens).sum()
        if world > 1:
            dist.all_reduce(den)
            for p in params:
                if p.grad is not None:
                    dist.all_reduce(p.grad)
        scale = torch.where(den > 0, args.accum / den.clamp_min(1e-6), torch.zeros_like(den))
        for p in params:
            if p.grad is not None:
                p.grad.mul_(scale.to(p.grad.dtype))
        if opt is not None:
            opt.step()
        for p in params:
            p.grad = None
        return tokens

    def sync():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    for s in range(args.warmup):
        update(s)
    sync()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    tokens = 0
    for s in range(args.steps):
        tokens += update(args.warmup + s)
    if cuda:
        e1.record()
    sync()
    ms = e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3
    stats = torch.tensor([ms, float(tokens)], device=device, dtype=torch.float64)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(stats)
        ms, tokens = float(mx[0]), float(stats[1])
        dist.destroy_process_group()
    if rank != 0:
        return None
    value = tokens / (ms / 1e3)
    return {"impl": "reference", "metric": "Draft-only training input tokens/s, Qwen3-8B DSpark 4K", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / max(args.steps, 1), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / 15256.44, "dtype": "bf16" if cuda else "fp32", "data": "synthetic",
            "config": {"model": "Qwen3-8B-shaped DSpark draft, random init", "layers": args.layers,
                       "target_layers": n_tl, "block_size": 7, "num_anchors": 512, "docs_per_update_per_rank": args.accum,
                       "lengths": [args.min_len, args.max_len], "attention_backend": backend,
                       "parallelism": f"dp{world}", "l2_policy": "inputs larger than L2 (weights + head > 126 MB)"}}
