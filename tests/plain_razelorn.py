"""A plain, slow implementation of the Razelorn decoder: whole sequences, no cache, no batching, one function per
mechanism, written from the design's equations with plain tensor arithmetic. It shares no code with the engine and is
the oracle of its tests. All functions work in the type of the tensors they are given (float64 in the tests).

Notation: ``n`` tokens of one sequence, positions 0 .. n - 1; ``x`` is ``[n, width]``; a linear weight is ``[out, in]``
and applied as ``x @ W.T``; ``W`` maps tensor names to tensors; ``cfg`` is the ``config.json`` dictionary.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w + b


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict], dtype=torch.float64) -> torch.Tensor:
    """f_i = base^(-2 i / dims), i < dims / 2, then the wavelength-dependent rescaling: short waves are kept, long ones
    divided by ``factor``, and those between are blended linearly in original / wavelength."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = []
    for fi in f.tolist():
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            out.append(fi)
        elif wave > original / low:
            out.append(fi / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * fi / factor + s * fi)
    return torch.tensor(out, dtype=dtype)


def rotate_half(v: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """Rotation of the first 2 len(freq) entries of the last axis of ``v`` [n, ..., d]; entry i is paired with entry
    i + len(freq); the other entries pass."""
    half = freq.numel()
    if half == 0:
        return v
    angle = positions.to(v.dtype)[:, None] * freq.to(v.dtype)[None, :]
    while angle.dim() < v.dim():
        angle = angle.unsqueeze(1)
    cos, sin = torch.cos(angle), torch.sin(angle)
    a, b = v[..., :half], v[..., half:2 * half]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., 2 * half:]], dim=-1)


def two_map_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, window: Optional[int],
                      scale: float, lam: float, diff: float, eps: float) -> torch.Tensor:
    """q [n, H, 2, d], k [n, G, 2, d], v [n, G, dv] as they enter the scores (normed and rotated) -> [n, H dv]: per head
    two softmax maps over the visible keys, a1 - lam a2, divided by its root mean square, times 1 - diff."""
    n, H, G = q.shape[0], q.shape[1], k.shape[1]
    i, j = positions[:, None], positions[None, :]
    visible = (j <= i) if window is None else ((j <= i) & (i - j < int(window)))
    heads = []
    for head in range(H):
        g = head // (H // G)
        maps = []
        for which in range(2):
            score = (q[:, head, which] @ k[:, g, which].T) * scale
            score = score.masked_fill(~visible, float("-inf"))
            maps.append(torch.softmax(score, dim=-1) @ v[:, g])
        heads.append(rms(maps[0] - lam * maps[1], eps) * (1.0 - diff))
    return torch.cat(heads, dim=-1)


def map_factor(W: Dict[str, torch.Tensor], p: str, diff: float) -> torch.Tensor:
    return torch.exp((W[f"{p}.lq1"] * W[f"{p}.lk1"]).sum()) - torch.exp((W[f"{p}.lq2"] * W[f"{p}.lk2"]).sum()) + diff


def differential_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
                           positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Two softmax maps per head over the same values; the second is subtracted with a learned factor, the difference
    is divided by its root mean square and scaled by 1 - diff."""
    n = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    positions = torch.arange(n) if positions is None else positions
    q = (h @ W[f"{p}.q"].T).view(n, H, 2, d)
    k = (h @ W[f"{p}.k"].T).view(n, G, 2, d)
    v = (h @ W[f"{p}.v"].T).view(n, G, dv)
    q = rms(q, eps) * W[f"{p}.q.norm"]
    k = rms(k, eps) * W[f"{p}.k.norm"]
    rot = m.get("rot")
    if rot and int(rot.get("dims", 0)) > 0:
        freq = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"), h.dtype)
        q, k = rotate_half(q, positions, freq), rotate_half(k, positions, freq)
    window = (m.get("mask") or {}).get("size")
    heads = two_map_attention(q, k, v, positions, window, float(m["scale"]), float(map_factor(W, p, diff)), diff, eps)
    return heads @ W[f"{p}.o"].T


def dense_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    z = torch.relu(h @ W[f"{p}.up"].T)
    return (z * z) @ W[f"{p}.down"].T


def gated_expert(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    g = h @ W[f"{p}.gate"].T
    return ((g * torch.sigmoid(g)) * (h @ W[f"{p}.up"].T)) @ W[f"{p}.down"].T


def route(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, top: int):
    """(chosen expert ids [n, top], their weights [n, top]): softmax scores over all router outputs, the choice by
    score + correction, the weight the plain score."""
    s = torch.softmax(h @ W[f"{p}.router"].T, dim=-1)
    choice = s + W[f"{p}.correction"] if f"{p}.correction" in W else s
    ids = torch.topk(choice, top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def expert_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    router = mlp["router"]
    E, identity, top = int(router["experts"]), int(router.get("identity", 0) or 0), int(router["top"])
    ids, weights = route(h, W, p, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t].tolist(), weights[t]):
            if e >= E:
                assert e < E + identity
                out[t] += w * h[t]
            else:
                out[t] += w * gated_expert(h[t:t + 1], W, f"{p}.e{e}")[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ W[f"{p}.shared.sg"].T)                   # [n, 1]
        out = out + gate * gated_expert(h, W, f"{p}.shared")
    return out


def owner(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else int(j)


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [n, vocab] of one sequence. ``residuals``: a list that receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{owner(cfg, i)}"
        h = layer_norm(x, W[f"{p}.norm1"], W[f"{p}.norm1.b"], eps)
        delta = differential_attention(h, W, f"{p}.mix", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            delta = delta + (dense_ff(h, W, f"{p}.mlp") if mlp["kind"] == "dense" else expert_ff(h, W, f"{p}.mlp", mlp))
        x = x + delta
        if residuals is not None:
            residuals.append(x)
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
