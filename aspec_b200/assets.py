"""Locates bundled recipes and draft configs (reference: aspec/assets.py)."""
from __future__ import annotations

import os

_ROOT = os.path.dirname(os.path.abspath(__file__))


def asset_dirs():
    return [os.path.join(_ROOT, "config", "drafts"), os.path.join(_ROOT, "config"), os.path.join(_ROOT, "recipes"),
            os.path.join(os.path.dirname(_ROOT), "configs")]


def find_asset(name: str) -> str:
    if os.path.exists(name):
        return name
    for d in asset_dirs():
        for cand in (os.path.join(d, name), os.path.join(d, os.path.basename(name))):
            if os.path.exists(cand):
                return cand
    raise FileNotFoundError(f"asset {name!r} not found in {asset_dirs()}")
