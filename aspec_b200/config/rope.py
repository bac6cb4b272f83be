"""RoPE base / scaling resolution (default, linear, YaRN).

Behaviour of the reference's ``aspec/config/utils.py:62-227``: ``rope_theta`` may be
a top-level field or live inside ``rope_parameters``; a conflict between the two
is refused; DFlash-family GQA drafts support full-head static RoPE of type
default / linear / yarn only.
"""
from __future__ import annotations

import copy
import math
from typing import Any, Optional


def _get(config: Any, key: str, default=None):
    if isinstance(config, dict):
        return config.get(key, default)
    return getattr(config, key, default)


def resolve_rope_theta(config: Any, default: Optional[float] = 10000.0) -> Optional[float]:
    top = _get(config, "rope_theta")
    params = _get(config, "rope_parameters")
    nested = params.get("rope_theta") if isinstance(params, dict) else None
    if top is not None and nested is not None and float(top) != float(nested):
        raise ValueError(f"Conflicting rope_theta: attribute is {top} but rope_parameters carries {nested}")
    if top is not None:
        return float(top)
    if nested is not None:
        return float(nested)
    return None if default is None else float(default)


def resolve_rope_parameters(config: Any) -> dict:
    params = copy.deepcopy(_get(config, "rope_parameters") or _get(config, "rope_scaling") or {})
    kind = params.get("rope_type", params.get("type", "default"))
    if kind not in ("default", "linear", "yarn"):
        raise ValueError(f"DFlash/DSpark GQA RoPE type {kind!r} is not supported")
    if params.get("partial_rotary_factor", 1.0) != 1.0:
        raise ValueError("DFlash/DSpark GQA requires full-head RoPE")
    params.update(rope_type=kind, rope_theta=resolve_rope_theta(config))
    if kind != "default":
        f = params.get("factor")
        if isinstance(f, bool) or not isinstance(f, (int, float)) or not math.isfinite(f) or f <= 0:
            raise ValueError("RoPE scaling factor must be finite and positive")
    if kind == "yarn":
        params.setdefault("original_max_position_embeddings", _get(config, "max_position_embeddings"))
        orig = params["original_max_position_embeddings"]
        if type(orig) is not int or orig <= 0:
            raise ValueError("YaRN original_max_position_embeddings must be positive")
        for field in ("beta_fast", "beta_slow", "attention_factor"):
            v = params.get(field)
            if v is not None and (not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0):
                raise ValueError(f"YaRN {field} must be finite and positive")
    return params


def rope_inverse_frequencies(head_dim: int, params: dict):
    """Returns (inv_freq list[float] of length head_dim/2, attention scaling factor)."""
    theta = float(params.get("rope_theta") or 10000.0)
    half = head_dim // 2
    base = [theta ** (-(2.0 * i) / head_dim) for i in range(half)]
    kind = params.get("rope_type", "default")
    if kind == "default":
        return base, 1.0
    factor = float(params["factor"])
    if kind == "linear":
        return [f / factor for f in base], 1.0
    # YaRN: blend interpolated and extrapolated frequencies with a linear ramp between the
    # dimensions whose wavelength completes beta_fast / beta_slow rotations in the original window.
    orig = params["original_max_position_embeddings"]
    beta_fast = float(params.get("beta_fast") or 32.0)
    beta_slow = float(params.get("beta_slow") or 1.0)

    def corr_dim(n_rot):
        return (head_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), head_dim - 1)
    if low == high:
        high += 0.001
    out = []
    for i, f in enumerate(base):
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        extrap_w = 1.0 - ramp
        out.append((f / factor) * (1 - extrap_w) + f * extrap_w)
    att = params.get("attention_factor")
    if att is None:
        att = 0.1 * math.log(factor) + 1.0 if factor > 1 else 1.0
    return out, float(att)
