"""Target feature contract: what a producer (the in-framework Target, a replay engine) must deliver to a Draft
consumer - captured layers, tensor names, dtypes, shapes, value stage - hashed into a ``contract_id`` that travels
with every ring slot, offline dataset and checkpoint (reference: aspec/feature_contract.py:63-403).

Algorithm identity is not part of the contract: identical payloads stay shareable between Drafts
(``shared_feature_union`` builds the superset one Target pass must produce for several Drafts).
"""
from __future__ import annotations

import copy
import hashlib
import json
from typing import Any, Dict, List, Mapping, Sequence

import torch

FEATURE_CONTRACT_SCHEMA_VERSION = "aspec.target-feature-contract/v1"
PRODUCER = {"backend": "native_prefill", "mode": "prefill_only"}
TRANSPORT = "symmetric_ring"
_DTYPES = {"bfloat16": torch.bfloat16, "int64": torch.int64, "float32": torch.float32}


class FeatureContractError(ValueError):
    pass


def _contract_id(contract: Mapping[str, Any]) -> str:
    body = {k: v for k, v in contract.items() if k != "contract_id"}
    return hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def build_target_feature_contract(*, drafter_family: str, target_hidden_size: int, target_num_hidden_layers: int,
                                  aux_hidden_state_layers: Sequence[int], store_last_hidden_states: bool) -> Dict[str, Any]:
    layers = list(aux_hidden_state_layers)
    if not isinstance(target_hidden_size, int) or target_hidden_size <= 0:
        raise FeatureContractError(f"draft target_hidden_size must be a positive integer, got {target_hidden_size!r}")
    if not isinstance(target_num_hidden_layers, int) or target_num_hidden_layers <= 0:
        raise FeatureContractError(f"draft target_num_hidden_layers must be a positive integer, got {target_num_hidden_layers!r}")
    if not layers or not all(isinstance(i, int) and i >= 0 for i in layers):
        raise FeatureContractError(f"aux_hidden_state_layers must contain non-negative integers, got {layers!r}")
    if len(layers) != len(set(layers)):
        raise FeatureContractError(f"aux_hidden_state_layers must be unique and ordered explicitly, got {layers!r}")
    if max(layers) >= target_num_hidden_layers:
        raise FeatureContractError(f"aux_hidden_state_layers must be within the target decoder; max layer {max(layers)} "
                                   f">= {target_num_hidden_layers}")
    tensors: Dict[str, Any] = {
        "hidden_states": {"semantic": "selected_decoder_layer_outputs", "dtype": "bfloat16",
                          "shape": ["sequence", len(layers) * target_hidden_size], "layout": "layers_concatenated_last_dim"},
        "input_ids": {"semantic": "target_token_ids", "dtype": "int64", "shape": ["sequence"], "layout": "sequence"},
    }
    if drafter_family == "mtp":
        if len(layers) != 1 or store_last_hidden_states:
            raise FeatureContractError("Native MTP requests one post-norm feature, without a duplicate teacher tensor")
        tensors["hidden_states"] = {"semantic": "target_final_hidden_state", "dtype": "bfloat16",
                                    "shape": ["sequence", target_hidden_size], "layout": "sequence_hidden",
                                    "value_stage": "post_norm"}
    if store_last_hidden_states:
        tensors["last_hidden_states"] = {"semantic": "target_final_hidden_state", "dtype": "bfloat16",
                                         "shape": ["sequence", target_hidden_size], "layout": "sequence_hidden",
                                         "value_stage": "post_norm"}
        distribution, omissions = "consumer_lm_head_from_last_hidden_states", [{"tensor": "logits", "reason": "computed_by_consumer_lm_head"}]
    else:
        distribution, omissions = "token_labels", [{"tensor": "logits", "reason": "not_required_by_objective"}]
    contract: Dict[str, Any] = {
        "schema_version": FEATURE_CONTRACT_SCHEMA_VERSION, "producer": dict(PRODUCER),
        "consumer": {"target_distribution": distribution}, "transport": TRANSPORT,
        "target_hidden_size": target_hidden_size, "target_num_hidden_layers": target_num_hidden_layers,
        "aux_hidden_state_layers": layers, "tensors": tensors, "omissions": omissions}
    contract["contract_id"] = _contract_id(contract)
    return contract


def validate_feature_contract(contract: Mapping[str, Any]) -> None:
    if contract.get("schema_version") != FEATURE_CONTRACT_SCHEMA_VERSION:
        raise FeatureContractError(f"Unsupported target feature contract schema: {contract.get('schema_version')!r}")
    if contract.get("contract_id") != _contract_id(contract):
        raise FeatureContractError(f"Target feature contract identity mismatch: {contract.get('contract_id')!r} != "
                                   f"{_contract_id(contract)!r}")
    if contract.get("producer") != PRODUCER:
        raise FeatureContractError(f"Unsupported target feature producer contract: {contract.get('producer')!r}")
    if contract.get("transport") != TRANSPORT:
        raise FeatureContractError(f"Unsupported target feature transport: {contract.get('transport')!r}")
    if not isinstance(contract.get("tensors"), Mapping) or not contract["tensors"]:
        raise FeatureContractError("Target feature contract must declare tensors")


class FeatureContractRuntime:
    """Validates one participant's payloads against the shared contract and counts what it saw."""

    def __init__(self, contract: Mapping[str, Any], *, role: str, participant: str):
        validate_feature_contract(contract)
        if role not in ("producer", "consumer"):
            raise FeatureContractError(f"Unknown target feature participant role: {role!r}")
        self.contract = copy.deepcopy(dict(contract))
        self.role, self.participant = role, participant
        self.validated_payloads = 0
        self.validated_tokens = 0

    @property
    def contract_id(self) -> str:
        return self.contract["contract_id"]

    def validate_binding(self, other_contract_id: str) -> None:
        if other_contract_id != self.contract_id:
            raise FeatureContractError(f"{self.participant}: feature contract {other_contract_id!r} does not match "
                                       f"{self.contract_id!r}")

    def validate_payload(self, tensors: Mapping[str, torch.Tensor]) -> None:
        seq = None
        for name, spec in self.contract["tensors"].items():
            if name not in tensors:
                raise FeatureContractError(f"{self.participant}: payload is missing tensor {name!r}")
            t = tensors[name]
            if t.dtype != _DTYPES[spec["dtype"]]:
                raise FeatureContractError(f"{self.participant}: {name} has dtype {t.dtype}, contract says {spec['dtype']}")
            shape = list(t.shape[-len(spec["shape"]):])
            for dim, want in zip(shape, spec["shape"]):
                if want == "sequence":
                    if seq is not None and dim != seq:
                        raise FeatureContractError(f"{self.participant}: {name} sequence length {dim} != {seq}")
                    seq = dim
                elif dim != want:
                    raise FeatureContractError(f"{self.participant}: {name} has width {dim}, contract says {want}")
        extra = set(tensors) - set(self.contract["tensors"]) - {"loss_mask"}
        for omitted in self.contract["omissions"]:
            if omitted["tensor"] in extra:
                raise FeatureContractError(f"{self.participant}: payload carries omitted tensor {omitted['tensor']!r}")
        self.validated_payloads += 1
        self.validated_tokens += int(seq or 0)

    def audit(self) -> dict:
        return {"participant": self.participant, "role": self.role, "contract_id": self.contract_id,
                "validated_payloads": self.validated_payloads, "validated_tokens": self.validated_tokens}


def shared_feature_union(contracts: Sequence[Mapping[str, Any]]) -> Dict[str, Any]:
    """The one payload a shared Target must produce for several Drafts: ordered union of captured layers, the final
    hidden state if any reader wants it, and per-reader column views into the union."""
    if not contracts:
        raise FeatureContractError("shared_feature_union needs at least one contract")
    for c in contracts:
        validate_feature_contract(c)
    hidden = {c["target_hidden_size"] for c in contracts}
    depth = {c["target_num_hidden_layers"] for c in contracts}
    if len(hidden) != 1 or len(depth) != 1:
        raise FeatureContractError("Drafts that share a Target must agree on its width and depth")
    layers: List[int] = sorted({i for c in contracts for i in c["aux_hidden_state_layers"]})
    want_last = any("last_hidden_states" in c["tensors"] for c in contracts)
    union = build_target_feature_contract(drafter_family="shared", target_hidden_size=hidden.pop(),
                                          target_num_hidden_layers=depth.pop(), aux_hidden_state_layers=layers,
                                          store_last_hidden_states=want_last)
    views = [{"contract_id": c["contract_id"], "layer_columns": [layers.index(i) for i in c["aux_hidden_state_layers"]],
              "last_hidden_states": "last_hidden_states" in c["tensors"]} for c in contracts]
    return {"contract": union, "views": views}
