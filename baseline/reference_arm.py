"""Reference arm of the benchmark: the unmodified reference package (installed under ``baseline/_ref``) runs the
same Draft-only workload through its own public API and stock code path.

Preferred driver, the one the reference's own Draft-only benchmark uses
(tools/performance/dspark_draft_benchmark.py:199-340): ``DSparkTrainer(Namespace(...))`` ->
``init_model(draft_config, target_path)`` -> a resident document feed in place of the queue fetcher ->
``train_from_queue(step, num_batches)`` per optimizer update (aspec/training/trainer.py:539-760,
aspec/training/dflash_trainer.py:489-533,747-806, aspec/training/fsdp.py:147-231).  ``init_model`` reads the Target's
embedding and output head from a checkpoint directory, so the arm first writes a random-init Qwen3-8B-shaped one
(``config.json`` + ``model.safetensors`` with the three tensors it reads) to a temporary directory.

If that driver cannot be set up on this image (the reference pins torch 2.13; this image has 2.11) the arm falls
back to the reference's model / optimizer classes driven by a restatement of its update loop
(``backward(numerator / accumulation)`` per micro-batch, gradients scaled by ``accumulation / sum(denominators)``)
and says so in ``config.driver``.

Nothing from ``aspec_b200`` is on the timed path; only the synthetic documents are shared so that both arms see
identical shapes.  Attention backends are tried in the reference's own order of preference (``fa4``,
``cudnn_flex_attention``, then ``flex_attention``); the one that ran is printed.

Two numbers, like the other arm: ``value`` with the documents resident on the GPU, ``e2e.value`` with every
micro-batch copied from pinned host memory inside the timed region and the update's metrics read back.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
METRIC = "Draft input tokens/s, Qwen3-8B DSpark 4K (Draft-only, resident features)"


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


def _dims(args):
    if args.small:
        return dict(hidden_size=256, intermediate_size=512, num_attention_heads=2, num_key_value_heads=1,
                    head_dim=128, vocab_size=4096, target_hidden_size=256, markov_rank=32, mask_token_id=4095)
    return dict(hidden_size=4096, intermediate_size=12288, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, vocab_size=151936, target_hidden_size=4096, markov_rank=256, mask_token_id=151669)


def _pick_backend() -> tuple:
    """The reference's backends in its own order of preference; the first whose library imports is used."""
    forced = os.environ.get("ASPEC_REFERENCE_ATTENTION_BACKEND")
    if forced:
        return forced, [f"{forced} (forced by ASPEC_REFERENCE_ATTENTION_BACKEND)"]
    tried = []
    try:
        import flash_attn.cute  # noqa: F401
        return "fa4", ["fa4: flash_attn.cute importable"]
    except Exception as exc:
        tried.append(f"fa4: {type(exc).__name__}")
    try:
        import cudnn
        if not hasattr(cudnn, "flex_attention") and not hasattr(getattr(cudnn, "pygraph", None), "flex_attention"):
            raise ImportError("cudnn frontend lacks flex_attention")
        return "cudnn_flex_attention", tried + ["cudnn_flex_attention: importable"]
    except Exception as exc:
        tried.append(f"cudnn_flex_attention: {type(exc).__name__}")
    return "flex_attention", tried + ["flex_attention: torch"]


def _write_target_checkpoint(path: str, dims: dict, device) -> None:
    """A random-init Qwen3-shaped checkpoint holding only what ``init_model`` reads."""
    import torch
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": dims["hidden_size"],
           "intermediate_size": dims["intermediate_size"], "num_hidden_layers": 36,
           "num_attention_heads": dims["num_attention_heads"], "num_key_value_heads": dims["num_key_value_heads"],
           "head_dim": dims["head_dim"], "vocab_size": dims["vocab_size"], "rms_norm_eps": 1e-6, "rope_theta": 1e6,
           "max_position_embeddings": 40960, "tie_word_embeddings": False, "torch_dtype": "bfloat16"}
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    g = torch.Generator(device=device).manual_seed(4321)
    V, H = dims["vocab_size"], dims["hidden_size"]
    tensors = {
        "model.embed_tokens.weight": (torch.randn(V, H, device=device, generator=g) * 0.02).bfloat16().cpu(),
        "lm_head.weight": (torch.randn(V, H, device=device, generator=g) * 0.02).bfloat16().cpu(),
        "model.norm.weight": torch.ones(H, dtype=torch.bfloat16),
    }
    save_file(tensors, os.path.join(path, "model.safetensors"))


def _documents(args, cfg_vocab, n_tl, target_hidden, rank, cuda):
    sys.path.insert(0, os.path.dirname(HERE))
    from aspec_b200.data.synthetic import SyntheticSpec, benchmark_documents, synthetic_features
    spec = SyntheticSpec(vocab_size=cfg_vocab - 1024, min_len=min(args.min_len, args.max_len),
                         max_len=args.max_len, seed=17)
    n_docs = args.pool or args.accum * 2
    pool = []
    for doc in benchmark_documents(spec, n_docs, args.accum, rank):
        feats = synthetic_features(doc["seq_len"], n_tl, target_hidden, doc["row"], pin=cuda)
        ids, lm = doc["input_ids"][None], doc["loss_mask"][None]
        if cuda:
            ids, lm = ids.pin_memory(), lm.pin_memory()
        pool.append({"input_ids": ids, "loss_mask": lm, "hidden_states": feats["hidden_states"][None],
                     "last_hidden_states": feats["last_hidden_states"][None], "seq_len": doc["seq_len"]})
    return pool, n_docs


class _Feed:
    """Stands where the queue fetcher stands: an iterator of micro-batches (aspec/training/trainer.py:760)."""

    def __init__(self, source, accum, n_docs, device, copy):
        self.source, self.accum, self.n_docs, self.device, self.copy = source, accum, n_docs, device, copy
        self.cursor = 0

    def seek(self, step):
        self.cursor = step * self.accum

    def __iter__(self):
        return self

    def __next__(self):
        import torch
        b = self.source[self.cursor % self.n_docs]
        self.cursor += 1
        out = {k: (v.to(self.device, non_blocking=True) if self.copy else v) for k, v in b.items() if torch.is_tensor(v)}
        return out


def _stock_trainer(args, dims, n_tl, ids, backend, device, rank, world):
    """Build the reference's own DSpark trainer the way its Draft-only benchmark does."""
    import argparse
    import dataclasses

    import torch
    import torch.distributed as dist
    from aspec.config import train_config as ref_config
    from aspec.training.dspark_trainer import DSparkTrainer
    from aspec.utils.distributed import init_gloo_group
    defaults = {**dataclasses.asdict(ref_config.TrainingConfig()), **dataclasses.asdict(ref_config.DebugConfig())}
    target_dir = os.path.join(tempfile.gettempdir(), f"aspec_ref_target_{'small' if args.small else 'qwen3_8b'}")
    if rank == 0 and not os.path.exists(os.path.join(target_dir, "model.safetensors")):
        _write_target_checkpoint(target_dir, dims, device)
    dist.barrier()
    defaults.update(
        target_model_path=target_dir, chat_template=None, attention_backend=backend, draft_context_parallel_size=1,
        dflash_packing=False, micro_batch_size=1, draft_accumulation_steps=args.accum, max_seq_length=args.max_len,
        dspark_num_anchors=512 if not args.small else 64, dspark_num_target_layers=n_tl, dflash_block_size=7,
        dspark_loss_decay_gamma=4.0, dspark_ce_loss_alpha=0.1, dspark_l1_loss_alpha=0.9,
        dspark_confidence_head_alpha=1.0, learning_rate=6e-4, min_lr=6e-5, max_grad_norm=1.0, weight_decay=0.0,
        warmup_ratio=0.04, lr_total_steps=max(args.steps * 2 + args.warmup * 2 + 8, 32),
        # the reference's own Draft-only benchmark settings (tools/performance/dspark_draft_benchmark.py:235-236)
        fsdp_strategy="FULL_SHARD", fsdp_reduce_dtype="bfloat16", last_hidden_states_prenorm=False, load_path=None,
        resume=None, seed=731, enable_perf_metrics=True, checkpoint_dir=None)
    init_gloo_group()
    trainer = DSparkTrainer(argparse.Namespace(**defaults))
    draft_config = dict(architectures=["DSparkDraftModel"], num_hidden_layers=args.layers, num_target_layers=n_tl,
                        target_layer_ids=ids, target_num_hidden_layers=36, rope_theta=1e6,
                        max_position_embeddings=40960, rms_norm_eps=1e-6, **dims)
    trainer.init_model(draft_config, target_dir)
    return trainer


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

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dtype = torch.bfloat16 if cuda else torch.float32
    dims = _dims(args)
    n_tl = args.target_layers
    ids = {3: [2, 18, 33], 5: [1, 9, 17, 25, 33]}.get(n_tl)
    backend, tried = _pick_backend()

    trainer, driver, why_not = None, None, None
    if cuda:
        if not dist.is_initialized():
            if world == 1:
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", str(29400 + os.getpid() % 500))
                os.environ.setdefault("RANK", "0")
                os.environ.setdefault("WORLD_SIZE", "1")
            dist.init_process_group("nccl", device_id=device)
        try:
            trainer = _stock_trainer(args, dims, n_tl, ids, backend, device, rank, world)
            driver = "stock DSparkTrainer.init_model + train_from_queue (the reference's own Draft-only benchmark driver)"
        except Exception as exc:                                   # noqa: BLE001 - reported in the JSON line
            why_not = f"{type(exc).__name__}: {str(exc)[:200]}"
        # every rank must take the same path
        ok = torch.tensor([1 if trainer is not None else 0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if not int(ok):
            trainer = None
    elif world > 1:
        dist.init_process_group("gloo")

    pool, n_docs = _documents(args, dims["vocab_size"], n_tl, dims["target_hidden_size"], rank, cuda)
    resident = [{k: (v.to(device) if torch.is_tensor(v) else v) for k, v in b.items()} for b in pool]

    if trainer is not None:
        feeds = {"resident": _Feed(resident, args.accum, n_docs, device, copy=False),
                 "host": _Feed(pool, args.accum, n_docs, device, copy=True)}

        def update(step: int, source: str, read: bool) -> int:
            feed = feeds[source]
            feed.seek(step)
            trainer.data_fetcher = feed
            metrics = trainer.train_from_queue(step=step, num_batches=args.accum)
            if read and metrics is not None:
                float(metrics.get("train/avg_loss", 0.0))
            return sum(pool[(step * args.accum + m) % n_docs]["seq_len"] for m in range(args.accum))
    else:
        update = _restated_loop(args, dims, n_tl, ids, backend, device, dtype, world, cuda, pool, resident, n_docs)
        driver = "reference DSparkModel / BF16Optimizer classes under a restated update loop" + (
            f" (stock trainer unavailable: {why_not})" if why_not else " (no GPU)")

    def sync():
        if world > 1 or (cuda and dist.is_initialized()):
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def timed(source: str, read: bool):
        for s in range(args.warmup):
            update(s, source, read)
        sync()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        tokens = 0
        for s in range(args.steps):
            tokens += update(args.warmup + s, source, read)
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
        return ms, tokens

    ms, tokens = timed("resident", read=False)
    e2e = None
    if not getattr(args, "no_e2e", False):
        ms2, tokens2 = timed("host", read=True)
        h2d = sum(v.numel() * v.element_size() for m in range(args.accum)
                  for v in pool[(args.warmup * args.accum + m) % n_docs].values() if torch.is_tensor(v))
        e2e = {"value": tokens2 / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4, "ms_per_step": ms2 / max(args.steps, 1)}
    if dist.is_initialized():
        dist.destroy_process_group()
    if rank != 0:
        return None
    value = tokens / (ms / 1e3)
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": (value / 15256.44) if world == 1 else None,
            "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (uniform token ids, log-uniform lengths, random bf16 features, random-init weights)",
            "e2e": e2e,
            "config": {"model": f"Qwen3-8B-shaped DSpark draft, {args.layers} layer(s), {n_tl} captured layers, vocab {dims['vocab_size']}",
                       "global_batch": args.accum * world, "seq_len": args.max_len,
                       "doc_lengths": f"log-uniform [{args.min_len},{args.max_len}]", "parallelism": f"dp{world}",
                       "micro_batch": "1 document (MBS1)", "anchors": 512 if not args.small else 64, "block_size": 7,
                       "attention_backend": backend, "backends_tried": tried, "driver": driver,
                       "anchors_sampled": "inside the timed region, every micro-batch (the model's own sampler)",
                       "l2_policy": "inputs larger than L2 (weights + head > 126 MB)"}}


def _restated_loop(args, dims, n_tl, ids, backend, device, dtype, world, cuda, pool, resident, n_docs):
    """Fallback driver: the reference's model and optimizer classes, its accumulation-window normalisation restated
    (aspec/training/dflash_trainer.py:489-533)."""
    import torch
    import torch.distributed as dist
    from aspec.models.draft.dspark import DSparkConfig, DSparkDraftModel
    from aspec.models.dspark import DSparkModel
    from aspec.training.optimizer import BF16Optimizer
    cfg = DSparkConfig(num_hidden_layers=args.layers, num_target_layers=n_tl, target_layer_ids=ids,
                       target_num_hidden_layers=36, rope_theta=1e6, max_position_embeddings=40960,
                       rms_norm_eps=1e-6, **dims)
    torch.manual_seed(1234)
    draft = DSparkDraftModel(cfg).to(device=device, dtype=dtype)
    model = DSparkModel(draft, block_size=7, num_anchors=512 if not args.small else 64, loss_decay_gamma=4.0,
                        ce_loss_alpha=0.1, l1_loss_alpha=0.9, confidence_head_alpha=1.0, attention_backend=backend)
    model.train()
    lm_head = (torch.randn(cfg.vocab_size, cfg.hidden_size, device=device, dtype=torch.float32) * 0.02).to(dtype)
    opt = BF16Optimizer(draft, lr=1e-4, weight_decay=0.0, max_grad_norm=0.5, total_steps=100000) if cuda else None
    params = [p for p in draft.parameters() if p.requires_grad]

    def update(step: int, source: str, read: bool) -> int:
        tokens = 0
        dens, nums = [], []
        docs = resident if source == "resident" else pool
        for m in range(args.accum):
            b = docs[(step * args.accum + m) % n_docs]
            dev = {k: v.to(device, non_blocking=True) for k, v in b.items() if torch.is_tensor(v)}
            out = model(dev["input_ids"], dev["hidden_states"].to(dtype), dev["loss_mask"], lm_head,
                        last_hidden_states=dev["last_hidden_states"].to(dtype))
            num, den = out[6]
            (num / args.accum).backward()
            dens.append(den.detach().float())
            nums.append(num.detach().float())
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
        if read:
            float(torch.stack(nums).sum() / den.clamp_min(1e-6))
        return tokens

    return update
