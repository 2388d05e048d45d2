"""Recurrent mixers: a fixed-size state per request instead of a cache that grows.

``min_gru`` is a gated recurrence whose gate and candidate read the current token only, so that the recurrence is
linear in its state. With h the mixer's input and W the state's width::

    z = sigmoid(Wz h + bz)                   the gate
    u = Wx h + bx,  c = u + 1/2 if u >= 0 else sigmoid(u)      the candidate (positive, continuous at 0)
    S_t = (1 - z) S_(t-1) + z c              element by element, S = 0 before the first token
    out = Wo (S_t * silu(Wg h))

The three input products are one matrix product against [Wz; Wx; Wg] with a float32 result; gate, candidate, state
and the recurrence are float32 (``csrc/min_gru.cu``), the gated state is rounded to the compute type for the output
product, whose result is float32 again. The state lives in the request's slot of the cache manager as two vectors that
take turns (a step of one token never overwrites the vector it read), so a captured decode step can be replayed."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import StateSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("min_gru")
class MinGRU(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, width: int):
        self.prefix, self.hidden_size, self.width = prefix, int(hidden_size), int(width)
        self.w_in = self.bias = self.w_out = None

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((2, self.width), torch.float32)

    def graph_key_group(self):
        return "min_gru"                      # its launches for a step of single tokens depend on the number of requests alone

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, W = self.prefix, self.hidden_size, self.width
        return {f"{p}.z": ParamSpec((W, H)), f"{p}.z.b": ParamSpec((W,), role="vector", init="small"),
                f"{p}.x": ParamSpec((W, H)), f"{p}.x.b": ParamSpec((W,), role="vector", init="small"),
                f"{p}.g": ParamSpec((W, H)), f"{p}.o": ParamSpec((H, W))}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_in = torch.cat([get(f"{p}.{n}", "matrix") for n in ("z", "x", "g")], dim=0).contiguous()
        self.bias = torch.cat([get(f"{p}.{n}.b", "vector").float() for n in ("z", "x")]).contiguous()
        self.w_out = get(f"{p}.o", "matrix").contiguous()

    def forward(self, x, ctx, cache: LayerCache):
        if cache.state is None:
            raise RuntimeError("the minGRU mixer needs its state slots")
        products = linear(x, self.w_in, out_dtype=torch.float32)
        gated = torch.empty((ctx.num_tokens, self.width), dtype=x.dtype, device=x.device)
        kernels.min_gru(products, self.bias, ctx.q_start, ctx.slots, ctx.positions, cache.state, gated, ctx.max_q_len)
        return linear(gated, self.w_out, out_dtype=torch.float32), None
