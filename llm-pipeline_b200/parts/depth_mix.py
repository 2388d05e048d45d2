"""Mixing over depth: what a layer hands on is a weighted sum of the results of all layers so far.

With X_0 the embedding's output and X_(i+1) the result of layer i, the layer hands on ``sum_j w[j] X_j`` over
j = 0 .. i + 1, with a learned weight vector ``w`` of its own (i + 2 entries). The sums are float32. The part only
holds the weights; the residual stream keeps the results (``ResidualStream.history``) and the next norm kernel takes
the sum while it has the row in hand (``ResidualStream.mix``)."""

from __future__ import annotations

from typing import Dict, Optional

from ..weights.source import ParamSpec
from .base import DepthMix, TensorGetter
from .registry import register_depth_mix


@register_depth_mix("weighted_average")
class DepthWeightedAverage(DepthMix):
    graph_safe = True

    def __init__(self, prefix: str, count: int, name: Optional[str] = None):
        """``count``: results that are summed (this layer's is the last of them)."""
        if count < 1:
            raise ValueError(f"a depth mix sums at least one result, got {count}")
        self.prefix, self.count, self.index = prefix, int(count), int(count) - 1
        self.name = name or f"{prefix}.weight"
        self.weights = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.count,), role="vector", init="average")}

    def load(self, get: TensorGetter) -> None:
        self.weights = get(self.name, "vector").float().contiguous()
