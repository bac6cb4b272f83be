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


def draft_catalog() -> dict:
    """``{name: raw Draft configuration}`` of the bundled catalog (``config/drafts/catalog.yaml``: per-target-model bases
    plus each configuration's own fields) together with the stand-alone ``config/drafts/*.json`` files."""
    import glob
    import json
    import yaml
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config", "drafts")
    out = {}
    path = os.path.join(root, "catalog.yaml")
    if os.path.exists(path):
        doc = yaml.safe_load(open(path)) or {}
        bases = doc.get("bases", {})
        for name, entry in (doc.get("configs") or {}).items():
            entry = dict(entry)
            base = entry.pop("base", None)
            out[name] = {**(bases[base] if base else {}), **entry}
    for p in sorted(glob.glob(os.path.join(root, "*.json"))):
        out[os.path.basename(p)[:-5]] = json.load(open(p))
    return out


def load_draft_config(name_or_path) -> dict:
    """A Draft configuration by file path, by bundled file name, or by catalog name (with or without ``.json``)."""
    import json
    if isinstance(name_or_path, dict):
        return dict(name_or_path)
    if os.path.exists(name_or_path):
        return json.load(open(name_or_path))
    key = os.path.basename(str(name_or_path))
    key = key[:-5] if key.endswith(".json") else key
    cat = draft_catalog()
    if key in cat:
        return cat[key]
    return json.load(open(find_asset(name_or_path)))
