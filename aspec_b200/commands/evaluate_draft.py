"""``evaluate``: acceptance statistics of an exported Draft on held-out documents, without a serving engine.

For every document a set of evaluation anchors is drawn deterministically; at each anchor the Draft proposes one
block through ``BlockDraftConsumer`` exactly as a speculative decoder would, and the proposal is verified greedily
against the document's own continuation (the tokens a Target that generated the document would accept).  Reports
per-position acceptance, the mean accepted length tau and the share of fully accepted blocks
(reference: aspec/commands/evaluate_draft.py, which drives a serving engine's decode loop for the same statistics).
Target features come from the in-framework Target (random-init unless weights are given) or an offline feature
dataset (``--features``)."""
from __future__ import annotations

import argparse
import json
import sys


def evaluate(consumer, lm_head, documents, features_of, *, anchors_per_doc: int = 16, seed: int = 0) -> dict:
    import torch
    bs = consumer.block_size
    accepted_at = torch.zeros(bs - 1)
    proposals = 0
    lengths = []
    g = torch.Generator().manual_seed(seed)
    for doc in documents:
        ids = doc["input_ids"].reshape(1, -1)
        T = ids.shape[1]
        if T < bs + 2:
            continue
        feats = features_of(doc)
        picks = torch.randperm(T - bs - 1, generator=g)[:anchors_per_doc] + 1
        for a in picks.tolist():
            out = consumer.propose(ids[:, : a + 1].to(feats.device), feats[:, : a + 1], lm_head_weight=lm_head)
            prop = out["token_ids"].reshape(-1)[: bs - 1].cpu()
            truth = ids[0, a + 1: a + bs]
            ok = (prop[: truth.numel()] == truth).long().cumprod(0)
            accepted_at[: ok.numel()] += ok.float()
            lengths.append(int(ok.sum()))
            proposals += 1
    if not proposals:
        return {"proposals": 0}
    rate = (accepted_at / proposals).tolist()
    return {"proposals": proposals, "accept_rate_at": rate, "tau": 1.0 + sum(lengths) / proposals,
            "mean_accepted_draft_tokens": sum(lengths) / proposals,
            "fully_accepted_share": sum(1 for n in lengths if n == bs - 1) / proposals}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec-b200 evaluate", description=__doc__)
    ap.add_argument("--asset-dir", required=True, help="directory written by `aspec-b200 export --format aspec`")
    ap.add_argument("--data", help="held-out conversations or pre-tokenised .jsonl (default: the documents of --features, "
                                   "or --synthetic N)")
    ap.add_argument("--synthetic", type=int, default=0, metavar="N", help="evaluate on N synthetic documents instead of --data")
    ap.add_argument("--features", "--feature-dir", dest="features",
                    help="offline feature dataset directory (else the in-framework Target computes them)")
    ap.add_argument("--target-weights")
    ap.add_argument("--tokenizer")
    ap.add_argument("--chat-template", default="qwen")
    ap.add_argument("--max-seq-length", type=int, default=4096)
    ap.add_argument("--block-size", type=int, default=7)
    ap.add_argument("--anchors-per-doc", type=int, default=16)
    ap.add_argument("--max-docs", type=int, default=256)
    ap.add_argument("--generate", type=int, default=0, metavar="N",
                    help="also run the speculative decode loop: from each document's prompt (the tokens before its first "
                         "supervised position) generate N tokens with the live Target and report tokens per Target pass")
    ap.add_argument("--generate-docs", type=int, default=16)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--output")
    a = ap.parse_args(argv)
    import torch
    from aspec_b200.data.dataset import load_training_samples
    from aspec_b200.draft_artifact import BlockDraftConsumer, load_native_draft
    dev = torch.device(a.device if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    draft, manifest = load_native_draft(a.asset_dir, device=dev, dtype=dtype)
    consumer = BlockDraftConsumer(draft, block_size=a.block_size)
    cfg = draft.config
    store = None
    if a.features:
        from aspec_b200.offline.dataset import OfflineFeatureStore
        store = OfflineFeatureStore(a.features)
    if a.data:
        docs = load_training_samples(a.data, {"tokenizer_path": a.tokenizer, "chat_template": a.chat_template,
                                              "max_seq_length": a.max_seq_length})[: a.max_docs]
    elif a.synthetic > 0:
        from aspec_b200.data.synthetic import SyntheticSpec, make_document
        limit = min(a.max_seq_length, int(getattr(cfg, "max_position_embeddings", a.max_seq_length) or a.max_seq_length))
        spec = SyntheticSpec(vocab_size=int(cfg.vocab_size) - 16, min_len=min(64, limit // 2), max_len=min(1024, limit), seed=20240229)
        docs = [make_document(spec, i) for i in range(a.synthetic)]
    elif store is not None:
        # the store's own documents, in the order they were written
        docs = []
        for row in list(store.rows("train"))[: a.max_docs]:
            rec = store.load(row["data_id"])
            docs.append({"data_id": row["data_id"], "input_ids": rec["input_ids"], "packed_loss_mask": rec["packed_loss_mask"]})
    else:
        ap.error("one of --data, --synthetic N or --features is needed")
    if store is not None:
        import os
        head_path = os.path.join(a.features, "lm_head.pt")      # optional: written next to the features by the generator
        lm_head = torch.load(head_path, map_location=dev).to(dtype) if os.path.exists(head_path) else None
        features_of = lambda d: store.load(d["data_id"])["hidden_states"][None].to(dev, dtype)
    else:
        from aspec_b200.inference.factory import target_config_from_args
        from aspec_b200.models.target.dense import DenseTarget, TargetConfig
        tcfg = target_config_from_args({"target_model_config": None}, cfg.to_dict())
        torch.set_default_dtype(dtype)
        with torch.device(dev):
            target = DenseTarget(TargetConfig(**tcfg))
        torch.set_default_dtype(torch.float32)
        if a.target_weights:
            target.load_state_dict(torch.load(a.target_weights, map_location=dev), strict=True)
        else:
            target.init_random(0)
        target.eval()
        layers = list(cfg.target_layer_ids or draft.target_layer_ids)
        lm_head = target.lm_head.detach()
        features_of = lambda d: target.prefill(d["input_ids"].reshape(-1).to(dev), [int(d["input_ids"].numel())], layers)["hidden_states"][None]
    if lm_head is None:
        raise ValueError("this offline feature dataset has no lm_head.pt; compute features with the in-framework Target instead (omit --features)")
    res = evaluate(consumer, lm_head, docs, features_of, anchors_per_doc=a.anchors_per_doc)
    res.update(asset=a.asset_dir, algorithm=manifest.get("algorithm"), documents=len(docs), block_size=a.block_size)
    if a.generate > 0:
        if a.features:
            raise ValueError("--generate needs the live Target (omit --features)")
        from aspec_b200.data.utils import unpack_loss_mask
        from aspec_b200.inference.speculative_decode import speculative_generate
        rounds, tokens, passes = [], 0, 0
        for d in docs[: a.generate_docs]:
            ids = d["input_ids"].reshape(-1)
            mask = unpack_loss_mask(d["packed_loss_mask"], ids.numel(), dtype=torch.bool)
            first = int(mask.float().argmax()) if bool(mask.any()) else ids.numel() // 2
            if first < 2:
                continue
            out = speculative_generate(target, consumer, ids[:first].to(dev), layers, max_new_tokens=a.generate)
            rounds += out["accepted_per_round"]
            tokens += len(out["tokens"])
            passes += out["target_passes"]
        res["generation"] = {"documents": min(len(docs), a.generate_docs), "new_tokens": tokens, "target_passes": passes,
                             "tokens_per_target_pass": tokens / max(passes, 1),
                             "mean_accepted_draft_tokens": sum(rounds) / max(len(rounds), 1)}
    text = json.dumps(res, indent=2)
    if a.output:
        open(a.output, "w").write(text + "\n")
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
