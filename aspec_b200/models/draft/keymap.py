"""Parameter-name mapping between the training layout and the serving export layout.

Export renames ``midlayer. -> layers.0.``, ``context_proj. -> fc.``, ``context_norm. -> hidden_norm.``,
``final_norm. -> norm.`` (reference: aspec/models/draft/keymap.py:27-68).  The inverse is not injective
across families, so a key is only renamed back when the model does not already own it.
"""
from __future__ import annotations

from typing import Collection, Dict

DRAFT_WEIGHT_KEY_REMAP = [("midlayer.", "layers.0."), ("context_proj.", "fc."),
                          ("context_norm.", "hidden_norm."), ("final_norm.", "norm.")]


def to_export_keys(tensors: Dict[str, object]) -> Dict[str, object]:
    out = {}
    for key, value in tensors.items():
        new = key
        for internal, exported in DRAFT_WEIGHT_KEY_REMAP:
            if key.startswith(internal):
                new = exported + key[len(internal):]
                break
        out[new] = value
    return out


def to_internal_keys(tensors: Dict[str, object], model_keys: Collection[str]) -> Dict[str, object]:
    model_keys = set(model_keys)
    out = {}
    for key, value in tensors.items():
        new = key
        if key not in model_keys:
            for internal, exported in DRAFT_WEIGHT_KEY_REMAP:
                if key.startswith(exported):
                    cand = internal + key[len(exported):]
                    if cand in model_keys:
                        new = cand
                        break
        out[new] = value
    return out
