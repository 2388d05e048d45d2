"""A plain, slow implementation of the Zupilorn decoder: whole sequences, no cache, no batching, one function per
mechanism, written from the design's equations with plain tensor arithmetic. It shares no code with the engine and is
the oracle of its tests. All functions work in the type of the tensors they are given (float64 in the tests).

Notation: ``n`` tokens of one sequence, positions 0 .. n - 1; ``x`` is ``[n, width]``; a linear weight is ``[out, in]``
and applied as ``x @ W.T``; ``W`` maps tensor names to tensors.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the stored weight lies around zero and stands for 1 + w."""
    return rms(x, eps) * (1.0 + w)


def plain_weight_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def rotate_half(v: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Rotary encoding of the first ``dims`` entries of the last axis of ``v`` [n, ..., d]: entry i is paired with
    entry i + dims / 2, angle = position * base^(-2 i / dims); entries from ``dims`` on pass unchanged."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]              # [n, half]
    while angle.dim() < v.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def min_gru(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, state: Optional[torch.Tensor] = None):
    """The gated recurrence whose gates read the current token only. Returns (output [n, width], last state)."""
    z = torch.sigmoid(h @ W[f"{p}.z"].T + W[f"{p}.z.b"])
    u = h @ W[f"{p}.x"].T + W[f"{p}.x.b"]
    candidate = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros_like(z[0]) if state is None else state
    states = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * candidate[t]
        states.append(s)
    g = h @ W[f"{p}.g"].T
    out = (torch.stack(states) * (g * torch.sigmoid(g))) @ W[f"{p}.o"].T
    return out, s


def latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict, eps: float) -> torch.Tensor:
    """Causal softmax attention whose keys and values are made from one small latent vector per token, plus one
    rotated key part that all heads share."""
    n = h.shape[0]
    H, d, r, dv, rank = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"], cfg["kv_rank"]
    rot = cfg["rot"]
    pos = torch.arange(n)
    q = (h @ W[f"{p}.q"].T).view(n, H, d + r)
    q_plain, q_rot = q[..., :d], rotate_half(q[..., d:], pos, rot["dims"], rot["base"])
    dkv = h @ W[f"{p}.dkv"].T
    c = plain_weight_norm(dkv[:, :rank], W[f"{p}.dkv.norm"], eps)
    k_rot = rotate_half(dkv[:, rank:], pos, rot["dims"], rot["base"])   # [n, r], one for all heads
    k_plain = (c @ W[f"{p}.uk"].T).view(n, H, d)
    v = (c @ W[f"{p}.uv"].T).view(n, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihr,jr->hij", q_rot, k_rot)) * cfg["scale"]
    visible = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhv->ihv", weights, v).reshape(n, H * dv)
    return out @ W[f"{p}.o"].T


def poly_norm(z: torch.Tensor, act: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = act[0], act[1], act[2], act[3]
    return a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e


def dense_feed_forward(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    return poly_norm(h @ W[f"{p}.up"].T, W[f"{p}.act"], eps) @ W[f"{p}.down"].T


def expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ W[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ W[f"{p}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[f"{p}.down"].T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen experts [n, top], their weights [n, top]): sigmoid scores, the largest ``top``, not renormalised."""
    s = torch.sigmoid(h @ W[f"{p}.router"].T)
    weights, chosen = torch.topk(s, top, dim=-1)
    return chosen, weights


def routed_feed_forward(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, cfg: dict) -> torch.Tensor:
    chosen, weights = route(h, W, p, cfg["router"]["top"])
    out = torch.zeros(h.shape[0], W[f"{p}.e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for k in range(chosen.shape[1]):
            e = int(chosen[t, k])
            out[t] += expert(weights[t, k] * h[t:t + 1], W, f"{p}.e{e}", cfg["expert"]["limit"])[0]      # the weight scales the input
    return out


def forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], layer_results: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence. ``layer_results``, if given, receives what goes on after every layer."""
    eps = config["norm"]["eps"]
    table = W["embed"]
    x = zero_centred_norm(table[torch.tensor(tokens)], W["embed.norm"], eps)
    results = [x]                                    # X_0, then every layer's result before the depth average
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}"
        h = zero_centred_norm(x, W[f"{p}.norm1"], eps)
        if layer["type"] == "mingru":
            m, _ = min_gru(h, W, f"{p}.mix")
        elif layer["type"] == "latent_attention":
            m = latent_attention(h, W, f"{p}.mix", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + zero_centred_norm(m, W[f"{p}.norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = zero_centred_norm(x, W[f"{p}.norm2"], eps)
            f = dense_feed_forward(h, W, f"{p}.mlp", eps) if mlp["kind"] == "dense" else routed_feed_forward(h, W, f"{p}.mlp", mlp)
            x = x + zero_centred_norm(f, W[f"{p}.norm2b"], eps)
        results.append(x)
        dwa = W[f"{p}.dwa"]
        x = sum(dwa[j] * results[j] for j in range(i + 2))
        if layer_results is not None:
            layer_results.append(x)
    logits = zero_centred_norm(x, W["final.norm"], eps) @ table.T
    cap = config["logit_softcap"]
    return cap * torch.tanh(logits / cap)
