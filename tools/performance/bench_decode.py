"""Decode micro-benchmark of the in-framework Target (the producer side of train with decode): ``--sequences`` prompts
of ``--prompt`` tokens are continued by ``--new`` tokens each, all sequences sharing every Target pass, keys and values
cached.

``python -m tools.performance.bench_decode [--sequences 32] [--prompt 512] [--new 128] [--draft ASSET_DIR] [--small]
[--device cuda|cpu]`` prints one JSON line: generated tokens per second, Target passes and tokens per pass (above 1 only
with ``--draft``, a native DSpark / DFlash asset whose blocks are verified), the prompt pass apart from the decode
passes, and - on a GPU - what fraction of the weight-streaming bound the decode passes reach: a pass over few rows has
to read every weight once, so its floor is ``weight bytes / copy bandwidth`` (``MEASURED_PEAKS.json`` at the repository
root when present, else 6.65 TB/s).  Times are CUDA events on a GPU and the host clock on the CPU; the model is the
Qwen3-8B shape with random weights (``--small``: a toy shape that runs anywhere).
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch


def _copy_bandwidth():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sequences", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--draft", default=None)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    from aspec_b200.inference.speculative_decode import batched_generate
    from aspec_b200.models.target.dense import DenseTarget, TargetConfig
    cuda = a.device.startswith("cuda")
    shape = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                 vocab_size=512) if a.small else {}
    if a.small:
        a.sequences, a.prompt, a.new = min(a.sequences, 4), min(a.prompt, 24), min(a.new, 12)
    dtype = torch.bfloat16 if cuda else torch.float32
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(a.device):
            target = DenseTarget(TargetConfig(**shape))
    finally:
        torch.set_default_dtype(prev)
    target.init_random(0).eval()
    consumer, layers = None, ()
    if a.draft:
        from aspec_b200.draft_artifact import BlockDraftConsumer, load_native_draft
        model, manifest = load_native_draft(a.draft, device=a.device, dtype=dtype)
        block = int(manifest.get("training_contract", {}).get("block_size") or getattr(model.config, "block_size", 0))
        consumer, layers = BlockDraftConsumer(model, block_size=block), tuple(model.config.target_layer_ids)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, target.config.vocab_size, (a.prompt,), generator=g) for _ in range(a.sequences)]

    def clock():
        if cuda:
            torch.cuda.synchronize()
        return time.perf_counter()

    def run(new_tokens):
        t0 = clock()
        out = batched_generate(target, prompts, max_new_tokens=[new_tokens] * a.sequences, temperature=a.temperature,
                               seeds=list(range(a.sequences)), consumer=consumer, layer_ids=layers)
        return clock() - t0, out

    run(2)                                               # warm-up: allocations, kernel attributes
    t_prompt, _ = run(1)                                 # the prompt pass alone yields every sequence's first token
    t_all, out = run(a.new)
    tokens = sum(len(o["tokens"]) for o in out)
    passes = max(o["target_passes"] for o in out)
    decode_s = max(t_all - t_prompt, 1e-9)
    result = {"bench": "decode", "device": a.device, "sequences": a.sequences, "prompt_tokens": a.prompt, "new_tokens": a.new,
              "draft": bool(consumer), "generated_tokens": tokens, "target_passes": passes,
              "tokens_per_pass_per_sequence": round(tokens / a.sequences / max(passes, 1), 3),
              "prompt_pass_ms": round(t_prompt * 1e3, 3), "decode_ms": round(decode_s * 1e3, 3),
              "generated_tokens_per_s": round((tokens - a.sequences) / decode_s, 1),
              "ms_per_decode_pass": round(decode_s * 1e3 / max(passes - 1, 1), 4)}
    if cuda:
        gbs, kind = _copy_bandwidth()
        floor_ms = target.memory_bytes() / (gbs * 1e9) * 1e3
        result.update(weight_bytes=target.memory_bytes(), weight_streaming_floor_ms=round(floor_ms, 4),
                      fraction_of_floor=round(floor_ms / max(result["ms_per_decode_pass"], 1e-9), 3), peaks=kind)
    print(json.dumps(result))
    return result


if __name__ == "__main__":
    main()
