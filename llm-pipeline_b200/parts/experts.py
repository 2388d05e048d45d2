"""A feed-forward of many small experts, of which every token uses a few.

With h the feed-forward's input, E experts and ``top`` of them per token::

    s = sigmoid(Wr h)                         router scores; the logits are float32
    chosen = the top experts by score; an expert's weight w is its score (not renormalised)
    expert_e(v): g = min(Wg_e v, limit), u = clamp(Wu_e v, -limit, limit), y = g sigmoid(1.702 g) (u + 1), Wd_e y
    out = sum over the chosen experts of expert_e(w h)       the weight scales the expert's input

``Wg_e (w h) = w (Wg_e h)``, so the weight is applied to the float32 sums of the first two products instead of making
a scaled copy of h per choice. Routing happens on the device (``csrc/routed_experts.cu``): nothing of a step depends on
the host seeing the choices, so the part can be captured in a CUDA graph. The experts' matrices are stacked:
``[E, 2 ff, hidden]`` (gate rows, then up rows) and ``[E, hidden, ff]``."""

from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from ..weights.source import ParamSpec
from .base import FeedForward, TensorGetter
from .registry import register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int, limit: float):
        if not 0 < top <= num_experts:
            raise ValueError(f"a token cannot use {top} of {num_experts} experts")
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.num_experts, self.top, self.limit = int(num_experts), int(top), float(limit)
        self.w_router = self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        specs = {f"{p}.router": ParamSpec((self.num_experts, H))}
        for e in range(self.num_experts):
            specs[f"{p}.e{e}.gate"] = ParamSpec((I, H))
            specs[f"{p}.e{e}.up"] = ParamSpec((I, H))
            specs[f"{p}.e{e}.down"] = ParamSpec((H, I))
        return specs

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_router = get(f"{p}.router", "matrix").float().contiguous()        # the logits are a 32-bit product
        self.w_gate_up = torch.stack([torch.cat([get(f"{p}.e{e}.gate", "matrix"), get(f"{p}.e{e}.up", "matrix")], dim=0)
                                      for e in range(self.num_experts)]).contiguous()
        self.w_down = torch.stack([get(f"{p}.e{e}.down", "matrix") for e in range(self.num_experts)]).contiguous()

    def forward(self, x, ctx):
        N = x.shape[0]
        ids = torch.empty((N, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((N, self.top), dtype=torch.float32, device=x.device)
        kernels.route_topk(x, self.w_router, self.top, ids, weights)
        out = torch.empty((N, self.hidden_size), dtype=torch.float32, device=x.device)
        kernels.routed_experts(x, self.w_gate_up, self.w_down, ids, weights, self.limit, out)
        return out, None
