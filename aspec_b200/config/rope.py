"""RoPE base / scaling resolution: default, linear, YaRN for every draft; llama3, dynamic NTK and
multi-axis (mrope) additionally for the EAGLE family.

Behaviour of the reference's ``aspec/config/utils.py:62-227``: ``rope_theta`` may be
a top-level field or live inside ``rope_parameters``; a conflict between the two
is refused; DFlash-family GQA drafts support full-head static RoPE of type
default / linear / yarn only (``resolve_rope_parameters``).  The EAGLE family also takes the
llama3, dynamic and mrope rules of ``aspec/models/draft/llama3_eagle.py:211-580``
(``rope_inverse_frequencies`` and ``mrope_axis_of_frequency`` below).
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
    if kind in ("default", "mrope"):
        # multi-axis RoPE uses the plain frequencies; which position axis feeds each one is mrope_axis_of_frequency
        return base, 1.0
    if kind == "llama3":
        return _llama3_frequencies(base, params), 1.0
    if kind == "dynamic":
        return _dynamic_ntk_frequencies(head_dim, theta, params), 1.0
    if kind not in ("linear", "yarn"):
        raise ValueError(f"Unknown RoPE scaling type {kind!r}")
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


def _llama3_frequencies(base, params: dict):
    """Llama-3.1 rule: wavelengths shorter than ``orig / high_freq_factor`` keep their frequency, those longer than
    ``orig / low_freq_factor`` are divided by ``factor``, and the band between is interpolated in wavelength."""
    factor = float(params.get("factor") or 1.0)
    low = float(params.get("low_freq_factor") or 1.0)
    high = float(params.get("high_freq_factor") or 4.0)
    orig = params.get("original_max_position_embeddings")
    if not orig or orig <= 0:
        raise ValueError("llama3 RoPE scaling needs original_max_position_embeddings")
    if high <= low:
        raise ValueError("llama3 RoPE scaling needs high_freq_factor > low_freq_factor")
    long_wave, short_wave = orig / low, orig / high
    out = []
    for f in base:
        wave = 2.0 * math.pi / f
        if wave < short_wave:
            out.append(f)
        elif wave > long_wave:
            out.append(f / factor)
        else:
            keep = (orig / wave - low) / (high - low)
            out.append((1.0 - keep) * f / factor + keep * f)
    return out


def _dynamic_ntk_frequencies(head_dim: int, theta: float, params: dict):
    """Dynamic NTK: once the row length exceeds the trained window the base grows so that the lowest frequency still
    spans the row.  Training rows have a fixed maximum, so the base is resolved once from ``sequence_length``
    (``max_seq_length`` of the run; the trained window when the key is absent, which leaves the base unchanged)."""
    factor = float(params["factor"])
    window = params.get("original_max_position_embeddings") or params.get("max_position_embeddings")
    if not window or window <= 0:
        raise ValueError("dynamic RoPE scaling needs the trained window (max_position_embeddings)")
    length = int(params.get("sequence_length") or window)
    if length > window:
        theta = theta * ((factor * length / window) - (factor - 1.0)) ** (head_dim / (head_dim - 2.0))
    return [theta ** (-(2.0 * i) / head_dim) for i in range(head_dim // 2)]


def mrope_axis_of_frequency(head_dim: int, mrope_section) -> list:
    """For multi-axis RoPE (temporal, height, width position streams): which stream rotates frequency ``i``.

    ``mrope_section`` lists how many consecutive frequencies each stream owns, cycling temporal / height / width; it
    must cover ``head_dim / 2`` frequencies.  Text tokens carry the same position on all three streams, for which the
    result equals ordinary RoPE."""
    sections = [int(x) for x in mrope_section]
    if any(x <= 0 for x in sections) or sum(sections) != head_dim // 2:
        raise ValueError(f"mrope_section {sections} must be positive and sum to head_dim / 2 = {head_dim // 2}")
    axes = []
    for j, width in enumerate(sections):
        axes.extend([j % 3] * width)
    return axes
