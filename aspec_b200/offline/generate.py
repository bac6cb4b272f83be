"""Materialise Target features to an offline dataset: run the in-framework Target (or any engine exposing
``features(input_ids) -> (hidden_states, last_hidden_states)``) over every document and append one record per
document (reference: aspec/offline/generate.py:156-308, aspec/offline/saving_actor.py:43-133)."""
from __future__ import annotations

import hashlib
import json
from typing import Callable, Dict, Iterable, Optional

import torch

from aspec_b200.data.utils import pack_loss_mask
from aspec_b200.feature_contract import build_target_feature_contract
from aspec_b200.offline.dataset import OfflineFeatureStore


def target_binding(target_identity: Dict, draft_config: Dict, family: str, store_last: bool) -> dict:
    layers = list(draft_config.get("target_layer_ids") or [])
    contract = build_target_feature_contract(
        drafter_family=family, target_hidden_size=int(draft_config["target_hidden_size"]),
        target_num_hidden_layers=int(draft_config["target_num_hidden_layers"]), aux_hidden_state_layers=layers,
        store_last_hidden_states=store_last)
    ident = hashlib.sha256(json.dumps(target_identity, sort_keys=True).encode()).hexdigest()
    return {"target_identity": target_identity, "target_identity_sha256": ident, "feature_contract": contract}


def materialize(output_dir: str, documents: Iterable[dict], features: Callable[[torch.Tensor], tuple], binding: dict,
                *, split: str = "train", resume: bool = False, progress: Optional[Callable[[int], None]] = None,
                lm_head: Optional[torch.Tensor] = None, embedding: Optional[torch.Tensor] = None) -> OfflineFeatureStore:
    """``documents`` yield ``{"data_id", "input_ids", "loss_mask"}``; ``features(ids)`` returns the contract's tensors.
    ``lm_head`` (the Target's frozen output head) and ``embedding`` (its token embedding, which Drafts borrow frozen)
    are saved beside the features as ``lm_head.pt`` / ``embed_tokens.pt`` in the Target's own dtype, so that training
    and decode evaluation from the dataset alone see the model that made the features."""
    store = (OfflineFeatureStore(output_dir, allow_incomplete=True) if resume
             else OfflineFeatureStore(output_dir, create=True, binding=binding, last_hidden_states_prenorm=False))
    if resume and store.binding["feature_contract"]["contract_id"] != binding["feature_contract"]["contract_id"]:
        raise ValueError("Cannot resume materialisation under a different Target feature contract")
    done = {r["data_id"] for r in store.rows(split)}
    want_last = "last_hidden_states" in binding["feature_contract"]["tensors"]
    for n, doc in enumerate(documents):
        data_id = str(doc.get("data_id", n))
        if data_id in done:
            continue
        ids = doc["input_ids"].reshape(-1).to(torch.int64)
        hidden, last = features(ids)
        rec = {"input_ids": ids.cpu(), "hidden_states": hidden.to(torch.bfloat16).cpu(),
               "packed_loss_mask": doc.get("packed_loss_mask") or pack_loss_mask(doc["loss_mask"].reshape(-1))}
        if want_last:
            rec["last_hidden_states"] = last.to(torch.bfloat16).cpu()
        store.append(split, data_id, rec)
        if progress:
            progress(n + 1)
    if lm_head is not None:
        import os
        torch.save(lm_head.detach().cpu(), os.path.join(output_dir, "lm_head.pt"))
    if embedding is not None:
        import os
        torch.save(embedding.detach().cpu(), os.path.join(output_dir, "embed_tokens.pt"))
    store.mark_complete()
    return store
