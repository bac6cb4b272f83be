"""Every bundled recipe loads, plans and names a Draft configuration that builds (meta device)."""
import glob
import json
import os

import pytest
import torch

import aspec_b200
from aspec_b200.config.draft_config import AutoDraftModelConfig, resolve_draft_algorithm
from aspec_b200.config.train_config import load_config
from aspec_b200.models.draft.auto import AutoEagle3DraftModel
from aspec_b200.planning import compile_execution_plan

ROOT = os.path.dirname(os.path.abspath(aspec_b200.__file__))
RECIPES = sorted(glob.glob(os.path.join(ROOT, "recipes", "*.yaml")))
from aspec_b200.assets import draft_catalog, load_draft_config

DRAFTS = sorted(draft_catalog())


@pytest.mark.parametrize("path", RECIPES, ids=[os.path.basename(p) for p in RECIPES])
def test_recipe_loads_and_plans(path):
    cfg = load_config(path, [])
    if cfg.experiments:
        from aspec_b200.multi_draft import compile_multi_draft_plan
        plan = compile_multi_draft_plan(cfg)
        assert len(plan.names) >= 2 and set(plan.plans) == set(plan.names)
        return
    plan = compile_execution_plan(cfg)
    flat = plan.to_runtime_args()
    assert flat["world_size"] >= 1 and plan.draft_config["architectures"]
    assert resolve_draft_algorithm(plan.draft_config) in ("dspark", "dflash", "dflash2", "eagle3", "eagle4", "mtp")


def test_the_catalog_covers_every_family():
    names = set(DRAFTS)
    assert len(names) >= 37
    for want in ("dspark_qwen3_8b_5layer", "dflash_base", "dflash2_qwen3_8b_swa", "eagle3_qwen3_8b_pruned", "eagle4_qwen3_8b_candidate",
                 "qwen3_5_9b_mtp", "dspark_qwen3_5_9b_dmtp", "dspark_ling3_flash_csa_sparse", "dspark_ling3_flash_qsa_indexer",
                 "dspark_qwen3_8b_dsa_sparse", "dspark_ling31_flash_mla_moe", "eagle3_qwen3_8b_mla", "dspark_qwen3_8_27b"):
        assert want in names, want
    assert load_draft_config("eagle3_qwen3_8b.json") == load_draft_config("eagle3_qwen3_8b")


@pytest.mark.parametrize("path", DRAFTS)
def test_bundled_draft_config_builds(path):
    raw = load_draft_config(path)
    cfg = AutoDraftModelConfig.from_dict(raw)
    with torch.device("meta"):
        model = AutoEagle3DraftModel.from_config(cfg)
    assert sum(p.numel() for p in model.parameters()) > 0
    again = AutoDraftModelConfig.from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()


def _plan(recipe, *overrides):
    return compile_execution_plan(load_config(os.path.join(ROOT, "recipes", recipe), list(overrides)))


@pytest.mark.parametrize("recipe,overrides,message", [
    ("qwen3_8b_dspark.yaml", ["training.training_num_gpus_per_node=8", "inference.inference_num_gpus=4"], "exceed the 8 GPUs"),
    ("qwen3_8b_dspark.yaml", ["inference.inference_engine_type=offline"], "feature_dir"),
    ("qwen3_8b_dspark.yaml", ["inference.inference_engine_type=remote_http"], "must be native, offline or synthetic"),
    ("qwen3_8b_dspark.yaml", ["training.training_num_nodes=2"], "training_num_nodes"),
    ("qwen3_8b_dspark.yaml", ["inference.inference_num_gpus=3", "inference.inference_num_gpus_per_engine=2"], "multiple of"),
    ("qwen3_8b_eagle3.yaml", ["training.sp_ulysses_size=3", "training.training_num_gpus_per_node=3"], "must divide the attention head counts"),
    ("qwen3_5_9b_mtp.yaml", ["training.sp_ring_size=2", "training.training_num_gpus_per_node=2"], "not sharded over sequences"),
    ("qwen3_8b_eagle3.yaml", ["training.eagle3_num_anchors=64"], "anchored EAGLE3"),
])
def test_the_planner_refuses_what_cannot_run(recipe, overrides, message):
    with pytest.raises(ValueError, match=message):
        _plan(recipe, *overrides)


def test_scope_notes_are_recorded_as_decisions():
    plan = _plan("qwen3_8b_dspark.yaml", "training.sp_ulysses_size=2", "training.training_num_gpus_per_node=2",
                 "inference.inference_num_gpus=1")
    notes = [c.reason for c in plan.capabilities if c.subsystem == "scope"]
    assert any("direct context parallelism" in n for n in notes)
    assert plan.policy["context_parallel"] == 2
    short = _plan("qwen3_8b_dspark.yaml", "debug.performance_measurement_required=true", "debug.performance_warmup_steps=4",
                  "debug.performance_drain_steps=2", "training.num_train_steps=6")
    assert any("needs more than 6 optimizer steps" in c.reason for c in short.capabilities if c.subsystem == "scope")
