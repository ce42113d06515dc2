"""Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.

Either side is any registered mixer, described like a layer's mixer (``{"kind", "params", "prefix"}``); each keeps the cache
it asks for, and this part asks for the pair.  The two outputs are float32 and the weighted sum is a 32-bit kernel.

Parameters: left, right (part descriptions), left_scale, right_scale.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from ..errors import require
from .base import build_part, register_part


def _spec(d) -> PartSpec:
    return d if isinstance(d, PartSpec) else PartSpec(str(d["kind"]), dict(d["params"]), str(d["prefix"]))


class ParallelMixers:
    can_overwrite = True

    def __init__(self, params, prefix: str):
        self.left = build_part("mixer", _spec(params["left"]))
        self.right = build_part("mixer", _spec(params["right"]))
        self.left_scale = float(params.get("left_scale", 1.0))
        self.right_scale = float(params.get("right_scale", 1.0))
        self.prefix = prefix

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False)) and bool(getattr(self.right, "graph_safe", False))

    def tensor_specs(self):
        return self.left.tensor_specs() + self.right.tensor_specs()

    def cache_requirement(self):
        return (self.left.cache_requirement(), self.right.cache_requirement())

    def bind(self, weights, ctx):
        self.left.bind(weights, ctx)
        self.right.bind(weights, ctx)

    def _side(self, part, h, batch, view, write_cache, like):
        fresh = bool(getattr(part, "can_overwrite", False))
        y = (torch.empty_like if fresh else torch.zeros_like)(like)
        part.forward(h, batch, view, y, write_cache, **({"overwrite": True} if fresh else {}))
        return y

    def forward(self, h, batch, cache_view, residual, write_cache=True, overwrite=False):
        require(isinstance(cache_view, tuple) and len(cache_view) == 2, f"{self.prefix}: two mixers need their two caches")
        l = self._side(self.left, h, batch, cache_view[0], write_cache, residual)
        r = self._side(self.right, h, batch, cache_view[1], write_cache, residual)
        if overwrite:
            ops.scaled_sum(self.left_scale, l, self.right_scale, r, residual)
        else:
            ops.scaled_sum(self.left_scale, l, self.right_scale, r, l)
            ops.scaled_sum(1.0, residual, 1.0, l, residual)
        return residual


register_part("mixer", "parallel", ParallelMixers)
