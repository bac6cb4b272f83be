"""Environment forwarded from the driver to actor processes: only an explicit allow-list of prefixes crosses, so a
run is reproducible from its recorded environment (reference: aspec/utils/env.py:23-89)."""
from __future__ import annotations

import os
from typing import Dict, Iterable, Mapping, Optional

FORWARD_PREFIXES = ("ASPEC_", "NCCL_", "CUDA_", "TORCH_", "OMP_", "HF_", "TOKENIZERS_")
FORWARD_EXACT = ("PATH", "LD_LIBRARY_PATH", "PYTHONPATH", "HOME", "TMPDIR", "MASTER_ADDR", "MASTER_PORT")
NEVER_FORWARD = ("CUDA_VISIBLE_DEVICES",)          # device selection is explicit per actor


def forwarded_environment(environ: Optional[Mapping[str, str]] = None, extra: Iterable[str] = ()) -> Dict[str, str]:
    environ = os.environ if environ is None else environ
    out = {}
    for k, v in environ.items():
        if k in NEVER_FORWARD:
            continue
        if k in FORWARD_EXACT or k in extra or k.startswith(FORWARD_PREFIXES):
            out[k] = v
    return out


def apply_environment(env: Mapping[str, str]) -> None:
    for k, v in env.items():
        os.environ[k] = v


def recorded_environment(environ: Optional[Mapping[str, str]] = None) -> Dict[str, str]:
    """What goes into ``evidence.json``: forwarded variables with secrets masked."""
    env = forwarded_environment(environ)
    return {k: ("***" if any(s in k.upper() for s in ("TOKEN", "KEY", "SECRET", "PASSWORD")) else v) for k, v in sorted(env.items())}
