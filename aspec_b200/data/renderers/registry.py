"""Renderer registry (reference: aspec/data/renderers/registry.py:26-57)."""
from __future__ import annotations

from typing import Any, Dict, List


class RendererRegistry:
    def __init__(self):
        self._renderers: Dict[str, type] = {}

    def register(self, name: str, renderer: type, override: bool = False) -> None:
        if not override and name in self._renderers:
            raise ValueError(f"renderer {name!r} is already registered")
        self._renderers[name] = renderer

    def get(self, name: str) -> type:
        if name not in self._renderers:
            raise KeyError(f"unknown renderer {name!r}; known: {sorted(self._renderers)}")
        return self._renderers[name]

    def create(self, name: str, tokenizer: Any):
        return self.get(name)(tokenizer)

    def cache_version(self, name: str) -> str:
        return str(getattr(self.get(name), "cache_version", "0"))

    def get_all_renderer_names(self) -> List[str]:
        return list(self._renderers)


RENDERER_REGISTRY = RendererRegistry()

from aspec_b200.data.renderers.kimi_k3 import K3Renderer  # noqa: E402

RENDERER_REGISTRY.register("kimi_k3", K3Renderer)
