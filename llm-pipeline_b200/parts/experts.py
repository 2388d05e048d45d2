"""A feed-forward of many small experts, of which every token uses a few.

With h the feed-forward's input, E experts with matrices, ``identity`` further router outputs without any, and ``top``
choices per token::

    z = Wr h                                  router logits, float32; one per expert and identity expert
    s = sigmoid(z)  or  softmax(z)            ``score``: each logit alone, or over all router outputs
    chosen = the top outputs by s (+ correction, a stored vector, if the router has one)
    an expert's weight w is its s (without the correction, not renormalised)
    expert_e(v), ``form`` "clamped": g = min(Wg_e v, limit), u = clamp(Wu_e v, -limit, limit), y = g sigmoid(1.702 g) (u + 1),
                                     Wd_e y, and the weight scales the expert's input: out += expert_e(w h)
                 ``form`` "silu":    Wd_e (silu(Wg_e v) (Wu_e v)), and the weight scales its output: out += w expert_e(h)
    an identity expert adds w h
    ``shared_size``: one more expert of the "silu" form that every token uses, added times sigmoid(w_sg . h)

The weight never makes a scaled copy: on the input side ``Wg_e (w h) = w (Wg_e h)`` puts it on the float32 sums of the
first two products, on the output side ``w (Wd_e y) = Wd_e (w y)`` puts it on the float32 activation. Routing happens on
the device (``csrc/routed_experts.cu``): nothing of a step depends on the host seeing the choices, so the part can be
captured in a CUDA graph. The experts' matrices are stacked: ``[E, 2 ff, hidden]`` (gate rows, then up rows) and
``[E, hidden, ff]``. The shared expert's gate is one more row of the float32 router matrix; its products are the
engine's ``linear`` and fused gate/up kernels."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import gate_up_swiglu, linear
from ..weights.source import ParamSpec
from .base import FeedForward, TensorGetter
from .registry import register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int, limit: float = 0.0,
                 score: str = "sigmoid", form: str = "clamped", identity: int = 0, correction: bool = False,
                 shared_size: Optional[int] = None):
        if not 0 < top <= num_experts + identity:
            raise ValueError(f"a token cannot use {top} of {num_experts + identity} experts")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"router scores are 'sigmoid' or 'softmax', not {score!r}")
        if form not in kernels.EXPERT_FORMS:
            raise ValueError(f"unknown expert form {form!r}; known: {sorted(kernels.EXPERT_FORMS)}")
        if num_experts < 1 or identity < 0:
            raise ValueError(f"{num_experts} experts and {identity} identity experts")
        self.prefix, self.hidden_size, self.intermediate_size = prefix, int(hidden_size), int(intermediate_size)
        self.num_experts, self.top, self.limit = int(num_experts), int(top), float(limit)
        self.score, self.form, self.identity, self.correction = score, form, int(identity), bool(correction)
        self.shared_size = int(shared_size) if shared_size else None
        self.w_router = self.w_gate_up = self.w_down = self.router_correction = self.w_shared_gate_up = self.w_shared_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        outputs = self.num_experts + self.identity
        specs = {f"{p}.router": ParamSpec((outputs, H))}
        if self.correction:
            specs[f"{p}.correction"] = ParamSpec((outputs,), role="vector", init="small")
        for e in range(self.num_experts):
            specs[f"{p}.e{e}.gate"] = ParamSpec((I, H))
            specs[f"{p}.e{e}.up"] = ParamSpec((I, H))
            specs[f"{p}.e{e}.down"] = ParamSpec((H, I))
        if self.shared_size:
            S = self.shared_size
            specs.update({f"{p}.shared.gate": ParamSpec((S, H)), f"{p}.shared.up": ParamSpec((S, H)),
                          f"{p}.shared.down": ParamSpec((H, S)), f"{p}.shared.sg": ParamSpec((1, H))})
        return specs

    def load(self, get: TensorGetter) -> None:
        p = self.prefix
        router = get(f"{p}.router", "matrix").float()                            # the logits are a 32-bit product
        if self.shared_size:
            router = torch.cat([router, get(f"{p}.shared.sg", "matrix").float().view(1, -1)], dim=0)
            self.w_shared_gate_up = torch.cat([get(f"{p}.shared.gate", "matrix"), get(f"{p}.shared.up", "matrix")], dim=0).contiguous()
            self.w_shared_down = get(f"{p}.shared.down", "matrix").contiguous()
        self.w_router = router.contiguous()
        if self.correction:
            self.router_correction = get(f"{p}.correction", "vector").float().contiguous()
        self.w_gate_up = torch.stack([torch.cat([get(f"{p}.e{e}.gate", "matrix"), get(f"{p}.e{e}.up", "matrix")], dim=0)
                                      for e in range(self.num_experts)]).contiguous()
        self.w_down = torch.stack([get(f"{p}.e{e}.down", "matrix") for e in range(self.num_experts)]).contiguous()

    def forward(self, x, ctx):
        N = x.shape[0]
        ids = torch.empty((N, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((N, self.top), dtype=torch.float32, device=x.device)
        gate = torch.empty((N,), dtype=torch.float32, device=x.device) if self.shared_size else None
        kernels.route_topk(x, self.w_router, self.top, ids, weights, softmax=self.score == "softmax",
                           correction=self.router_correction, gate=gate)
        out = torch.empty((N, self.hidden_size), dtype=torch.float32, device=x.device)
        kernels.routed_experts(x, self.w_gate_up, self.w_down, ids, weights, self.limit, out, self.form, self.identity)
        if self.shared_size:
            act = gate_up_swiglu(x, self.w_shared_gate_up)      # the few rows of a decode step: product and activation in one kernel
            if act is None:
                gate_up = linear(x, self.w_shared_gate_up)
                act = torch.empty((N, self.shared_size), dtype=x.dtype, device=x.device)
                kernels.swiglu(gate_up, act)
            kernels.add_scaled_rows(out, linear(act, self.w_shared_down, out_dtype=torch.float32), gate)
        return out, None
