"""Builds the Draft network and its training wrapper from a draft config and the flat run arguments
(the reference selects a trainer class per architecture: aspec/training/trainer_actor.py:42-72)."""
from __future__ import annotations

from typing import Any, Mapping

import torch

from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.models.draft.auto import AutoEagle3DraftModel


def build_training_model(draft_config, args: Mapping[str, Any], device, dtype) -> torch.nn.Module:
    cfg = draft_config if hasattr(draft_config, "to_dict") else AutoDraftModelConfig.from_dict(draft_config)
    algorithm = resolve_draft_algorithm(cfg.to_dict())
    g = args.get
    with torch.device(device):          # allocate and initialise on the target device, not through host memory
        draft = AutoEagle3DraftModel.from_config(cfg)
    draft = draft.to(dtype=dtype)
    if g("gradient_checkpointing"):
        draft.gradient_checkpointing = True
    common = dict(attention_backend=g("attention_backend", "sm100_flash"),
                  draft_context_parallel_size=g("draft_context_parallel_size", 1),
                  deterministic_anchor_sampling=g("deterministic_anchor_sampling", False),
                  anchor_seed=g("seed", 0), anchor_sampling_scope=g("anchor_sampling_scope", "row"))
    if algorithm == "dspark":
        from aspec_b200.models.dspark import DSparkModel
        return DSparkModel(draft, block_size=g("dspark_block_size", g("block_size", 7)),
                           num_anchors=g("dspark_num_anchors", 512), loss_decay_gamma=g("dspark_loss_decay_gamma", 4.0),
                           ce_loss_alpha=g("dspark_ce_loss_alpha", 0.1), l1_loss_alpha=g("dspark_l1_loss_alpha", 0.9),
                           confidence_head_alpha=g("dspark_confidence_head_alpha", 1.0),
                           l1_target_sampling=(g("dspark_l1_target_temperature", 1.0), g("dspark_l1_target_top_p", 1.0),
                                               g("dspark_l1_target_top_k", -1)),
                           l1_draft_sampling=(g("dspark_l1_draft_temperature", 1.0), g("dspark_l1_draft_top_p", 1.0),
                                              g("dspark_l1_draft_top_k", -1)), **common)
    if algorithm == "dflash":
        from aspec_b200.models.dflash import DFlashModel
        return DFlashModel(draft, block_size=g("dflash_block_size", 16), num_anchors=g("dflash_num_anchors", 512),
                           loss_objective=g("dflash_loss_objective", "decay"), dpace_alpha=g("dflash_dpace_alpha", 0.5),
                           loss_decay_gamma=g("dflash_loss_decay_gamma", 7.0), ce_loss_alpha=g("dflash_ce_loss_alpha", 1.0),
                           l1_loss_alpha=g("dflash_l1_loss_alpha", 0.0), **common)
    if algorithm == "dflash2":
        from aspec_b200.models.dflash2 import DFlash2Model
        return DFlash2Model(draft, block_size=g("dflash_block_size", 8), num_anchors=g("dflash_num_anchors", 512),
                            selector_loss_alpha=g("dflash2_selector_loss_alpha", 1.0), **common)
    if algorithm == "eagle3":
        from aspec_b200.models.eagle3 import Eagle3Model
        return Eagle3Model(draft, length=g("ttt_length", 7), loss_type=g("loss_type", "forward_kl"),
                           lk_eta=g("lk_eta", 3.0), ploss_weights=g("ploss_weights"))
    if algorithm == "eagle4":
        from aspec_b200.models.eagle4 import Eagle4TrainingModel
        draft.configure_training_stage()
        return Eagle4TrainingModel(draft, length=g("ttt_length", 7), loss_type=g("loss_type", "forward_kl"),
                                   lk_eta=g("lk_eta", 3.0), ploss_weights=g("ploss_weights"))
    if algorithm == "mtp":
        from aspec_b200.models.mtp import MTPModel
        return MTPModel(draft, length=g("mtp_steps", 3), step_weight_beta=g("mtp_step_weight_beta", 0.6))
    raise ValueError(f"no training wrapper for algorithm {algorithm!r}")
