"""Native Draft assets: validation, strict loading, and proposal-time consumers.

``validate_native_asset`` re-hashes ``config.json`` and ``model.safetensors`` against
``export_manifest.json`` and re-derives the algorithm before anything is allocated;
``load_native_draft`` loads strictly (no dropped indexer / head tensors).  ``BlockDraftConsumer``
proposes one block from a known prefix: the backbone runs once with a single anchor at the last token;
DFlash returns the argmax of slots ``1..bs-1``; DSpark decodes the block sequentially through the Markov
head only and also returns confidence logits.  Verification and acceptance belong to the caller
(reference: aspec/draft_artifact.py:58-286).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch
import torch.nn.functional as F

from aspec_b200.commands.convert_to_hf import SCHEMA, sha256_file
from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.models.draft.auto import AutoEagle3DraftModel


def validate_native_asset(asset_dir) -> dict:
    asset_dir = Path(asset_dir)
    manifest = json.loads((asset_dir / "export_manifest.json").read_text())
    if manifest.get("schema_version") != SCHEMA or manifest.get("storage_format") != "aspec_native":
        raise ValueError("not a native aspec asset (schema or storage format mismatch)")
    if sha256_file(asset_dir / "config.json") != manifest["config_sha256"]:
        raise ValueError("config.json does not match the export manifest")
    if sha256_file(asset_dir / "model.safetensors") != manifest["model_sha256"]:
        raise ValueError("model.safetensors does not match the export manifest")
    raw = json.loads((asset_dir / "config.json").read_text())
    if resolve_draft_algorithm(raw) != manifest["algorithm"]:
        raise ValueError("asset algorithm disagrees with its config")
    return manifest


def load_native_draft(asset_dir, *, device="cpu", dtype: Optional[torch.dtype] = None):
    """Returns ``(model, manifest)``; every tensor of the asset must be consumed and none may be missing."""
    from safetensors.torch import load_file
    asset_dir = Path(asset_dir)
    manifest = validate_native_asset(asset_dir)
    raw = json.loads((asset_dir / "config.json").read_text())
    raw = {k: v for k, v in raw.items() if k not in ("_aspec_version", "torch_dtype")}
    config = AutoDraftModelConfig.from_dict(raw)
    tensors = load_file(str(asset_dir / "model.safetensors"))
    if len(tensors) != manifest["tensor_count"]:
        raise ValueError("asset tensor count disagrees with its manifest")
    model = AutoEagle3DraftModel.from_config(config)
    model.load_state_dict(tensors, strict=True)
    if dtype is not None:
        model = model.to(dtype)
    return model.to(device).eval(), manifest


def write_live_asset(draft_model, output_dir, *, block_size: Optional[int] = None, source: str = "live weights") -> dict:
    """Write the weights a Draft holds RIGHT NOW as a native asset (same files and manifest fields as an export of a
    checkpoint), first under a temporary name and then renamed, so that a reader never sees half of it.  This is what a
    training run hands its decoding Target engines when it syncs weights
    (reference: weight sync to the serving engine, aspec/inference/engine/sgl_engine_decode.py:39-424)."""
    import os
    import shutil
    from safetensors.torch import save_file
    from aspec_b200 import __version__
    from aspec_b200.commands.convert_to_hf import draft_structure_manifest
    output_dir = Path(output_dir)
    staging = output_dir.with_name(output_dir.name + ".staging")
    if staging.exists():
        shutil.rmtree(staging)
    staging.mkdir(parents=True)
    raw = draft_model.config.to_dict()
    algorithm = resolve_draft_algorithm(raw)
    tensors = {k: v.detach().cpu().contiguous().clone() for k, v in draft_model.state_dict().items()}
    save_file(tensors, str(staging / "model.safetensors"), metadata={"format": "pt", "aspec_version": __version__})
    floats = [v.dtype for v in tensors.values() if v.is_floating_point()]
    dtype = max(set(floats), key=floats.count) if floats else torch.float32
    export_config = json.loads(json.dumps(raw))
    export_config.update(draft_vocab_size=int(raw.get("draft_vocab_size") or raw["vocab_size"]), _aspec_version=__version__,
                         torch_dtype=str(dtype).removeprefix("torch."))
    contract = {"algorithm": algorithm}
    if block_size:
        contract["block_size"] = export_config["block_size"] = int(block_size)
    (staging / "config.json").write_text(json.dumps(export_config, indent=2, sort_keys=True) + "\n")
    manifest = {"schema_version": SCHEMA, "storage_format": "aspec_native", "source_checkpoint": source,
                "model_sha256": sha256_file(staging / "model.safetensors"), "config_sha256": sha256_file(staging / "config.json"),
                "tensor_count": len(tensors), "dtype": str(dtype), "algorithm": algorithm, "training_contract": contract,
                "architecture": export_config.get("architectures"), "model_type": export_config.get("model_type"),
                "draft_structure": draft_structure_manifest(raw)}
    (staging / "export_manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    if output_dir.exists():
        shutil.rmtree(output_dir)
    os.replace(staging, output_dir)
    return manifest


class BlockDraftConsumer:
    def __init__(self, draft_model, *, block_size: int):
        from aspec_b200.models.dflash import DFlashModel
        self.model = draft_model.eval()
        if getattr(draft_model.config, "mtp_conditioning", None):
            raise ValueError("MTP-conditioned assets require an MTP-aware proposal consumer")
        self.algorithm = resolve_draft_algorithm(draft_model.config.to_dict())
        if self.algorithm not in ("dspark", "dflash"):
            raise ValueError("BlockDraftConsumer requires a DSpark or DFlash asset")
        if type(block_size) is not int or block_size < 2:
            raise ValueError("block_size must be an integer >= 2")
        saved = getattr(draft_model.config, "block_size", None)
        if saved is not None and saved != block_size:
            raise ValueError("Proposal block size disagrees with the trained asset")
        self.block_size = block_size
        self.backbone = DFlashModel(draft_model, block_size=block_size, num_anchors=1)

    @torch.no_grad()
    def update_weights_from_disk(self, asset_dir) -> dict:
        """Hot reload: validate a newer export of the same architecture and copy its tensors into the live modules in
        place, so compiled graphs, buffers and references held by a decode loop stay valid (the reference asks its
        serving engine for the same thing, aspec/inference/engine/sgl_engine_decode.py:39-424)."""
        from safetensors.torch import load_file
        asset_dir = Path(asset_dir)
        manifest = validate_native_asset(asset_dir)
        if manifest["algorithm"] != self.algorithm:
            raise ValueError("the new asset was trained with a different algorithm")
        tensors = load_file(str(asset_dir / "model.safetensors"))
        state = self.model.state_dict()
        if set(tensors) != set(state):
            raise ValueError("the new asset's tensor names differ from the loaded Draft")
        for name, t in tensors.items():
            if tuple(t.shape) != tuple(state[name].shape):
                raise ValueError(f"shape of {name} changed: {tuple(state[name].shape)} -> {tuple(t.shape)}")
        for name, t in tensors.items():
            state[name].copy_(t.to(state[name].device, state[name].dtype))
        return manifest

    @torch.no_grad()
    def propose(self, input_ids, target_features, *, lm_head_weight) -> dict:
        if input_ids.ndim != 2 or input_ids.shape[0] != 1 or input_ids.shape[1] < 1:
            raise ValueError("Block proposal currently consumes one nonempty prefix")
        L = input_ids.shape[1]
        cfg = self.model.config
        if tuple(target_features.shape) != (1, L, cfg.target_hidden_size * cfg.num_target_layers):
            raise ValueError("Target features must match the asset's ordered layers and prefix")
        if tuple(lm_head_weight.shape) != (cfg.vocab_size, cfg.hidden_size):
            raise ValueError("Frozen Target output head shape does not match the Draft")
        if L + self.block_size - 1 > cfg.max_position_embeddings:
            raise ValueError("Proposal exceeds the artifact's supported position range")
        dev = input_ids.device
        anchor = torch.tensor([[L - 1]])
        # the anchor is the last known token: its block sees the L-1 tokens before it
        hidden, _, _ = self.backbone._draft_backbone(
            input_ids, target_features, torch.ones(1, L, device=dev), injected_anchors=anchor,
            injected_keep_mask=torch.ones_like(anchor, dtype=torch.bool))
        if self.algorithm == "dflash":
            return {"token_ids": F.linear(hidden[1:], lm_head_weight).argmax(-1)[None], "algorithm": "dflash"}
        logits = F.linear(hidden, lm_head_weight)
        prev = input_ids[:, -1]
        markov, head = self.model.markov_head, self.model.confidence_head
        tokens, conf = [], []
        for j in range(self.block_size):
            row = logits[j:j + 1]
            if markov is not None:
                row = row + markov.compute_step_bias(prev).to(row.dtype)
            if head is not None:
                feats = hidden[j:j + 1]
                if self.model.confidence_head_with_markov:
                    feats = torch.cat((feats, markov.get_prev_embeddings(prev).to(feats.dtype)), -1)
                conf.append(head(feats))
            prev = row.argmax(-1)
            tokens.append(prev)
        out = {"token_ids": torch.stack(tokens, 1), "algorithm": "dspark"}
        if conf:
            out["draft_confidence_logits"] = torch.stack(conf, 1)
        return out
