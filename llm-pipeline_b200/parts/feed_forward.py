"""SwiGLU feed-forward: ``down(silu(gate(x)) * up(x))`` without biases
(src/llm_pipeline/models/qwen3/custom_builder.py:193-207; the activation is SiLU whatever
``hidden_act`` says, :204). Gate and up are one matrix product against [gate; up].
Beside it: ``poly_norm_mlp`` and ``relu_squared_mlp``, feed-forwards without a gate."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import PendingProduct, gate_up_swiglu, linear, pending_product
from ..weights.source import ParamSpec
from .base import FeedForward, TensorGetter
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, names: Optional[Dict[str, str]] = None):
        """``names``: the three matrices' names below ``prefix`` where they are not ``gate_proj.weight``, ``up_proj.weight``
        and ``down_proj.weight`` (keys ``gate``, ``up``, ``down``)."""
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I, n = self.prefix, self.hidden_size, self.intermediate_size, self.names
        return {f"{p}.{n['gate']}": ParamSpec((I, H)), f"{p}.{n['up']}": ParamSpec((I, H)), f"{p}.{n['down']}": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p, n = self.prefix, self.names
        self.w_gate_up = torch.cat([get(f"{p}.{n['gate']}", "matrix"), get(f"{p}.{n['up']}", "matrix")], dim=0).contiguous()
        self.w_down = get(f"{p}.{n['down']}", "matrix").contiguous()

    takes_scaled_rows = True             # x goes straight into gate_up_swiglu() or linear()

    def forward(self, x, ctx):
        out, bias = self.forward_deferred(x, ctx)
        return (out.value() if isinstance(out, PendingProduct) else out), bias

    def forward_deferred(self, x, ctx):
        act = gate_up_swiglu(x, self.w_gate_up)          # the few rows of a decode step: product and activation in one kernel
        if act is None:
            gate_up = linear(x, self.w_gate_up)
            act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.swiglu(gate_up, act)
        return pending_product(act, self.w_down), None


@register_feed_forward("poly_norm_mlp")
class PolyNormMLP(FeedForward):
    """``down(act(up(x)))`` without gate and biases, with the PolyNorm activation: for a token's vector z of ``ff``
    values, ``act(z) = a N(z) + b N(z^2) + c N(z^3) + e`` with powers taken element by element, N(v) = v / sqrt(mean(v^2)
    + eps) over the token's ff values, and the four learned numbers (a, b, c, e) in one tensor. The up product's result
    and the three mean squares are float32; the activation is rounded once to the compute type for the down product,
    whose result is float32."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, eps: float):
        self.prefix, self.hidden_size, self.intermediate_size, self.eps = prefix, int(hidden_size), int(intermediate_size), float(eps)
        self.w_up = self.w_down = self.act = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return {f"{p}.up": ParamSpec((I, H)), f"{p}.down": ParamSpec((H, I)), f"{p}.act": ParamSpec((4,), role="vector", init="unit")}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_up = get(f"{p}.up", "matrix").contiguous()
        self.w_down = get(f"{p}.down", "matrix").contiguous()
        self.act = get(f"{p}.act", "vector").float().contiguous()

    def forward(self, x, ctx):
        z = linear(x, self.w_up, out_dtype=torch.float32)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.poly_norm(z, self.act, self.eps, act)
        return linear(act, self.w_down, out_dtype=torch.float32), None


@register_feed_forward("relu_squared_mlp")
class ReluSquaredMLP(FeedForward):
    """``down(max(up(x), 0)^2)`` without gate and biases; the result is float32."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int):
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.w_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return {f"{p}.up": ParamSpec((I, H)), f"{p}.down": ParamSpec((H, I))}

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        self.w_up = get(f"{p}.up", "matrix").contiguous()
        self.w_down = get(f"{p}.down", "matrix").contiguous()

    def forward(self, x, ctx):
        z = linear(x, self.w_up)
        kernels.relu_squared(z, z)
        return linear(z, self.w_down, out_dtype=torch.float32), None
