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
DRAFTS = sorted(glob.glob(os.path.join(ROOT, "config", "drafts", "*.json")))


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


@pytest.mark.parametrize("path", DRAFTS, ids=[os.path.basename(p) for p in DRAFTS])
def test_bundled_draft_config_builds(path):
    raw = json.load(open(path))
    cfg = AutoDraftModelConfig.from_dict(raw)
    with torch.device("meta"):
        model = AutoEagle3DraftModel.from_config(cfg)
    assert sum(p.numel() for p in model.parameters()) > 0
    again = AutoDraftModelConfig.from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
