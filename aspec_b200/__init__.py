"""aspec_b200: B200-native training of speculative-decoding draft models.

Public names are resolved lazily (importing the package does not import torch models), mirroring the
reference's lazy exports (aspec/__init__.py:25-62).
"""
from __future__ import annotations

import importlib

__version__ = "0.2.0"

_EXPORTS = {
    "Eagle3Model": "aspec_b200.models.eagle3", "DFlashModel": "aspec_b200.models.dflash",
    "DFlashConfig": "aspec_b200.config.draft_config", "DFlashDraftModel": "aspec_b200.models.draft.dflash",
    "DFlash2Model": "aspec_b200.models.dflash2", "DFlash2Config": "aspec_b200.config.draft_config",
    "DFlash2DraftModel": "aspec_b200.models.draft.dflash2", "DSparkModel": "aspec_b200.models.dspark",
    "DSparkConfig": "aspec_b200.config.draft_config", "DSparkDraftModel": "aspec_b200.models.draft.dspark",
    "Eagle4TrainingModel": "aspec_b200.models.eagle4", "MTPModel": "aspec_b200.models.mtp",
    "AutoDraftModelConfig": "aspec_b200.config.draft_config", "AutoEagle3DraftModel": "aspec_b200.models.draft.auto",
}
__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
    module = _EXPORTS.get(name)
    if module is None:
        raise AttributeError(f"module 'aspec_b200' has no attribute {name!r}")
    return getattr(importlib.import_module(module), name)
