"""``aspec export``: training checkpoint -> ``model.safetensors`` + ``config.json`` + ``export_manifest.json``.

Reads the DCP model shards without a process group, strict-loads them into a freshly built Draft,
optionally remaps parameter names for serving (``--format sglang``) or keeps the native names
(``--format aspec``), and writes a manifest that binds config and weights by SHA-256
(reference: aspec/commands/convert_to_hf.py:336-515; schema ``aspec.serving-export/v1``).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import warnings
from collections import Counter
from pathlib import Path
from typing import Optional

import torch

from aspec_b200 import __version__
from aspec_b200.config.draft_attention import resolve_attention_policy, resolve_head_layout
from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.config.draft_structure import resolve_ffn_policy
from aspec_b200.models.draft.auto import AutoEagle3DraftModel
from aspec_b200.models.draft.keymap import to_export_keys

SCHEMA = "aspec.serving-export/v1"


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(8 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def detect_model_dir(input_dir: Path) -> Path:
    """Accepts a run dir, a ``checkpoints`` dir, an ``iter_N`` dir or the ``model`` dir itself."""
    if (input_dir / ".metadata").is_file():
        return input_dir
    if (input_dir / "model" / ".metadata").is_file():
        return input_dir / "model"
    for root in (input_dir, input_dir / "checkpoints"):
        tracker = root / "latest_checkpointed_iteration.txt"
        if tracker.is_file():
            return root / f"iter_{int(tracker.read_text().strip()):07d}" / "model"
    raise FileNotFoundError(f"model checkpoint not found under {input_dir}")


def load_dcp_state_dict(model_dir: Path) -> dict:
    from torch.distributed.checkpoint.state_dict_loader import _load_state_dict_from_keys
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        state = _load_state_dict_from_keys(checkpoint_id=str(model_dir))
    return state.get("model_state", state)


def draft_structure_manifest(raw: dict) -> dict:
    algorithm = resolve_draft_algorithm(raw)
    out = {"ffn": resolve_ffn_policy(raw) if algorithm != "mtp" else {"ffn_type": "dense"}}
    if algorithm != "mtp":
        policy = resolve_attention_policy(raw)
        out["attention"] = {"head_layout": resolve_head_layout(raw), "layer_types": policy["layer_types"],
                            "sliding_window": policy["sliding_window"], "window_semantics": policy["window_semantics"]}
    return out


def convert_checkpoint(*, input_dir: Path, output_dir: Path, config_path: Optional[Path] = None,
                       target_model_path: Optional[str] = None, output_dtype: Optional[torch.dtype] = None,
                       force: bool = False, artifact_format: str = "sglang") -> dict:
    if artifact_format not in ("sglang", "aspec"):
        raise ValueError("artifact_format must be sglang or aspec")
    input_dir = Path(input_dir).expanduser().resolve()
    output_dir = Path(output_dir).expanduser().resolve()
    model_dir = detect_model_dir(input_dir)
    ckpt_dir = model_dir.parent
    config_path = Path(config_path).resolve() if config_path else ckpt_dir / "draft_config.json"
    if not config_path.is_file():
        raise FileNotFoundError(f"draft config not found at {config_path}")
    if output_dir == ckpt_dir or ckpt_dir in output_dir.parents or output_dir in ckpt_dir.parents:
        raise ValueError("Export output directory must not overlap the source checkpoint or config")
    raw = json.loads(config_path.read_text())
    config = AutoDraftModelConfig.from_dict(raw)
    raw = config.to_dict()
    algorithm = resolve_draft_algorithm(raw)
    state = load_dcp_state_dict(model_dir)
    vocab, dvocab = int(raw["vocab_size"]), int(raw.get("draft_vocab_size") or raw["vocab_size"])
    vocabulary = None
    if dvocab != vocab:
        from aspec_b200.models.vocab import validate_vocab_mapping, vocab_mapping_manifest
        validate_vocab_mapping(state.get("d2t"), state.get("t2d"), dvocab, vocab)
        vocabulary = vocab_mapping_manifest(state["d2t"], state["t2d"])
    floats = Counter(v.dtype for v in state.values() if v.is_floating_point())
    ckpt_dtype = floats.most_common(1)[0][0]
    final_dtype = output_dtype or ckpt_dtype
    model = AutoEagle3DraftModel.from_config(config, torch_dtype=ckpt_dtype)
    missing, unexpected = model.load_state_dict(state, strict=False)
    allowed = {"embed_tokens.weight"} if target_model_path else set()
    bad_missing = sorted(set(missing) - allowed)
    if bad_missing or unexpected:
        raise RuntimeError("Checkpoint does not match the configured draft model: "
                           f"missing={bad_missing}, unexpected={sorted(unexpected)}")
    if final_dtype != ckpt_dtype:
        model = model.to(final_dtype)
    sd = model.state_dict()
    serving = sd if artifact_format == "aspec" else (
        model.state_dict_for_serving() if hasattr(model, "state_dict_for_serving") else to_export_keys(sd))
    tensors = {k: v.detach().cpu().contiguous().clone() for k, v in serving.items()}
    if output_dir.exists():
        if not force:
            raise FileExistsError(f"{output_dir} exists; pass -f to overwrite")
        shutil.rmtree(output_dir)
    output_dir.mkdir(parents=True)
    from safetensors.torch import save_file
    model_path = output_dir / "model.safetensors"
    save_file(tensors, str(model_path), metadata={"format": "pt", "aspec_version": __version__})
    export_config = json.loads(json.dumps(raw))
    export_config.update(draft_vocab_size=dvocab, _aspec_version=__version__,
                         torch_dtype=str(final_dtype).removeprefix("torch."))
    meta_path = ckpt_dir / "meta.json"
    contract = {"algorithm": algorithm}
    if meta_path.is_file():
        topo = json.loads(meta_path.read_text()).get("training_topology", {})
        contract.update(topo.get("training_objective", {}))
        if "block_size" in contract:
            export_config["block_size"] = contract["block_size"]
    cfg_out = output_dir / "config.json"
    cfg_out.write_text(json.dumps(export_config, indent=2, sort_keys=True) + "\n")
    manifest = {
        "schema_version": SCHEMA, "storage_format": "aspec_native" if artifact_format == "aspec" else "sglang",
        "source_checkpoint": str(model_dir), "source_config": str(config_path),
        "source_config_sha256": sha256_file(config_path), "model_sha256": sha256_file(model_path),
        "config_sha256": sha256_file(cfg_out), "tensor_count": len(tensors), "dtype": str(final_dtype),
        "algorithm": algorithm, "training_contract": contract, "architecture": export_config.get("architectures"),
        "model_type": export_config.get("model_type"), "draft_structure": draft_structure_manifest(raw),
        "vocabulary": vocabulary,
    }
    if algorithm == "eagle4":
        from aspec_b200.config.eagle4 import eagle4_asset_metadata
        manifest["eagle4"] = eagle4_asset_metadata(raw, int(getattr(model, "candidate_head_steps", 0)))
    if raw.get("mtp_conditioning"):
        from aspec_b200.config.mtp_conditioning import mtp_conditioning_semantics
        manifest["mtp_conditioning"] = mtp_conditioning_semantics(raw)
    if artifact_format == "aspec":
        block = algorithm in ("dspark", "dflash") and not raw.get("mtp_conditioning")
        mla = raw.get("architectures") == ["Eagle3DeepseekV2ForCausalLM"]
        manifest["draft_structure"]["loader_contract"] = {
            "runtime": "aspec_b200", "entrypoint": "aspec_b200.draft_artifact.load_native_draft",
            "proposal_entrypoint": ("aspec_b200.draft_artifact.MLAEagleConsumer" if mla else
                                    "aspec_b200.draft_artifact.BlockDraftConsumer" if block else None),
            "validation": "required_per_artifact",
            "borrowed_tensors": ["Target output head"] if algorithm in ("dspark", "dflash") else []}
    (output_dir / "export_manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    return manifest


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="aspec export", description=__doc__)
    ap.add_argument("--input-dir", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--format", default="sglang", choices=["sglang", "aspec"])
    ap.add_argument("--config")
    ap.add_argument("--target-model-path")
    ap.add_argument("--dtype", choices=["bfloat16", "float16", "float32"])
    ap.add_argument("-f", "--force", action="store_true")
    a = ap.parse_args(argv)
    manifest = convert_checkpoint(input_dir=Path(a.input_dir), output_dir=Path(a.output_dir),
                                  config_path=Path(a.config) if a.config else None,
                                  target_model_path=a.target_model_path,
                                  output_dtype=getattr(torch, a.dtype) if a.dtype else None,
                                  force=a.force, artifact_format=a.format)
    print(json.dumps({k: manifest[k] for k in ("storage_format", "algorithm", "tensor_count", "model_sha256")}, indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
