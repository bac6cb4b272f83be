"""Config -> Draft network registry (``AutoEagle3DraftModel.from_config``, aspec/models/draft/auto.py:43-64)."""
from __future__ import annotations

import importlib

from aspec_b200.config.draft_config import (AutoDraftModelConfig, DeepseekEagleConfig, DFlash2Config, DFlashConfig,
                                            DSparkConfig, Eagle3Config, Eagle4Config, K3DSparkConfig,
                                            NativeMTPConfig)

_MODEL_MAPPING = {
    Eagle3Config: ("aspec_b200.models.draft.llama3_eagle", "LlamaForCausalLMEagle3"),
    Eagle4Config: ("aspec_b200.models.draft.eagle4", "Eagle4DraftModel"),
    DeepseekEagleConfig: ("aspec_b200.models.draft.deepseek_eagle", "Eagle3DeepseekV2ForCausalLM"),
    NativeMTPConfig: ("aspec_b200.models.draft.mtp", "NativeMTPDraftModel"),
    DFlashConfig: ("aspec_b200.models.draft.dflash", "DFlashDraftModel"),
    DFlash2Config: ("aspec_b200.models.draft.dflash2", "DFlash2DraftModel"),
    DSparkConfig: ("aspec_b200.models.draft.dspark", "DSparkDraftModel"),
    K3DSparkConfig: ("aspec_b200.models.draft.dspark", "K3DSparkModel"),
}


class AutoEagle3DraftModel:
    @classmethod
    def model_class(cls, config):
        module, name = _MODEL_MAPPING[type(config)]
        return getattr(importlib.import_module(module), name)

    @classmethod
    def from_config(cls, config, torch_dtype=None, **kwargs):
        model = cls.model_class(config)(config, **kwargs)
        if torch_dtype is not None:
            model = model.to(dtype=torch_dtype)
        return model


__all__ = ["AutoDraftModelConfig", "AutoEagle3DraftModel"]
