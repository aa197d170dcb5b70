"""Two mixers side by side: both read the same input, and the result is a weighted sum of theirs,
``left_scale`` * left(h) + ``right_scale`` * right(h).

The two are parts of the mixer registry themselves (``left`` and ``right`` are ``PartSpec``s), with tensors under
``<prefix>.<left_name>`` and ``<prefix>.<right_name>``; each keeps what it keeps per sequence (the cache views arrive in the
order left, right).  Their results are products' float sums (or partial sums), added in float by one small kernel.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .base import DeferredProduct, Runtime, part_class, register_mixer


def _listed(request) -> list:
    if request is None:
        return []
    return list(request) if isinstance(request, (list, tuple)) else [request]


@register_mixer("side_by_side")
class SideBySide:
    def __init__(self, params, prefix: str, runtime: Runtime) -> None:
        self.prefix, self.runtime = prefix, runtime
        self.hidden = int(params["hidden_size"])
        self.scales = (float(params.get("left_scale", 1.0)), float(params.get("right_scale", 1.0)))
        self.parts = []
        for side in ("left", "right"):
            spec = params[side]
            self.parts.append(part_class("mixer", spec)(spec.params, f"{prefix}.{params.get(side + '_name', side)}", runtime))
        runtime.workspace.declare("side_by_side.out", runtime.max_step_tokens * self.hidden, torch.float32)

    @classmethod
    def expected_tensors(cls, params, prefix: str) -> dict:
        out = {}
        for side in ("left", "right"):
            spec = params[side]
            out.update(part_class("mixer", spec).expected_tensors(spec.params, f"{prefix}.{params.get(side + '_name', side)}"))
        return out

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts)

    def load(self, source) -> None:
        for part in self.parts:
            part.load(source)

    def cache_request(self):
        return [request for part in self.parts for request in _listed(part.cache_request())]

    def forward(self, x, ctx, cache):
        views = list(cache) if isinstance(cache, (list, tuple)) else [cache]
        results = []
        for part in self.parts:
            asked = part.cache_request()
            count = len(_listed(asked))
            mine, views = views[:count], views[count:]
            view = tuple(mine) if isinstance(asked, (list, tuple)) else (mine[0] if mine else None)
            result = part.forward(x, ctx, view)
            results.append(result.run() if isinstance(result, DeferredProduct) else result)
        tokens = x.shape[0]
        out = self.runtime.workspace.view("side_by_side.out", tokens, self.hidden)
        return kernels.weighted_sum(results[0], self.scales[0], results[1], self.scales[1], out)
