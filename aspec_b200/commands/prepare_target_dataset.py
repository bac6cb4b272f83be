"""``prepare-target-data``: materialise Target features for a tokenised corpus into an offline feature dataset
(``dataset.json`` + ``manifest.jsonl`` + ``samples/*.pt``) with the in-framework Target, so that Draft training can
run without Target GPUs (reference: aspec/commands/prepare_target_dataset.py, aspec/offline/generate.py:156-308)."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 prepare-target-data", description=__doc__)
    ap.add_argument("--input", required=True, help="conversations or pre-tokenised .jsonl")
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--draft-config", required=True)
    ap.add_argument("--target-config", help="Target config.json (default: shape-bound to the draft config)")
    ap.add_argument("--target-weights")
    ap.add_argument("--tokenizer")
    ap.add_argument("--chat-template", default="qwen")
    ap.add_argument("--max-seq-length", type=int, default=4096)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--split", default="train", choices=["train", "eval"])
    ap.add_argument("--resume", action="store_true")
    a = ap.parse_args(argv)
    import torch
    from aspec_b200.assets import load_draft_config
    from aspec_b200.config.draft_config import resolve_draft_algorithm
    from aspec_b200.data.dataset import load_training_samples
    from aspec_b200.inference.factory import target_config_from_args
    from aspec_b200.models.target.dense import DenseTarget, TargetConfig
    from aspec_b200.multi_draft import _layer_ids
    from aspec_b200.offline.generate import materialize, target_binding
    draft = load_draft_config(a.draft_config)
    algorithm = resolve_draft_algorithm(draft)
    layers = _layer_ids(draft)
    tcfg = (TargetConfig.from_file(a.target_config).to_dict() if a.target_config
            else target_config_from_args({"target_model_config": None}, draft))
    dev = torch.device(a.device if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.set_default_dtype(dtype)
    with torch.device(dev):
        target = DenseTarget(TargetConfig(**tcfg))
    torch.set_default_dtype(torch.float32)
    if a.target_weights:
        target.load_state_dict(torch.load(a.target_weights, map_location=dev), strict=True)
    else:
        target.init_random(0)
    target.eval()
    samples = load_training_samples(a.input, {"tokenizer_path": a.tokenizer, "chat_template": a.chat_template,
                                              "max_seq_length": a.max_seq_length})
    binding = target_binding({"config": tcfg, "weights": a.target_weights or "random-init seed 0"},
                             {**draft, "target_layer_ids": layers}, algorithm, store_last=algorithm != "mtp")

    def features(ids):
        out = target.prefill(ids.to(dev), [int(ids.numel())], layers)
        return out["hidden_states"], out["last_hidden_states"]

    docs = ({"data_id": s.get("data_id", i), "input_ids": s["input_ids"], "packed_loss_mask": s["packed_loss_mask"]}
            for i, s in enumerate(samples))
    store = materialize(a.output_dir, docs, features, binding, split=a.split, resume=a.resume, lm_head=target.lm_head,
                        embedding=target.embed_tokens.weight)
    print(json.dumps({"output_dir": a.output_dir, "samples": len(store), "contract_id": binding["feature_contract"]["contract_id"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
