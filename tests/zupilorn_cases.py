"""Small Zupilorn configurations with weights made for the tests, and the comparison with the plain implementation.

The weights are drawn so that every mechanism carries weight in the logits (projections of unit gain, biases and norm
weights well away from their neutral values, depth weights that keep old results alive) and are rounded to bfloat16
once, so the engine in either type and the float64 oracle read the same numbers. ``sharp`` scales the query
projections so that a softmax puts most of its weight on one or two keys, wherever they are: a key that is lost,
shifted by one or read from the wrong page then changes the result by its whole value, not by one part in hundreds.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

import plain_zupilorn as plain


def mingru_layer(width: int, mlp) -> dict:
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, mlp, base: float = 10000.0,
                 rot_dims: Optional[int] = None, scale: Optional[float] = None) -> dict:
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim),
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}},
            "mlp": mlp}


def dense(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def moe(experts: int, top: int, ff: int, limit: float = 1.5) -> dict:
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def config(layers: List[dict], width: int = 72, vocab: int = 211, eps: float = 1e-5, softcap: float = 9.0) -> dict:
    return {"architecture": "Zupilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": softcap,
            "layers": layers}


# Several shapes: other orders of layers, a layer without feed-forward, two recurrent layers in a row, one head, more
# experts per token than one, values of different size than keys, a latent that is no multiple of 32, widths that are
# no powers of two, a rotation of only a part of the rotated entries.
CONFIGS: Dict[str, dict] = {
    "hybrid": config([mingru_layer(96, dense(80)), latent_layer(3, 24, 8, 20, 40, moe(6, 2, 56)),
                      mingru_layer(56, moe(5, 1, 48, limit=0.75)), latent_layer(2, 16, 16, 24, 48, dense(104))]),
    "attention_first": config([latent_layer(4, 16, 8, 16, 36, dense(64), base=500000.0), mingru_layer(72, None),
                               mingru_layer(40, dense(96)), latent_layer(1, 32, 4, 40, 24, None, rot_dims=2)],
                              width=88, vocab=130, eps=3e-6, softcap=30.0),
    "dense_only": config([latent_layer(5, 8, 8, 8, 64, dense(72), base=1000.0), mingru_layer(64, dense(64)),
                          latent_layer(2, 40, 24, 12, 72, dense(40), scale=0.2)], width=64, vocab=97),
    # latents and rotated parts in multiples of 16 (the sizes of the tensor-core attention kernel in bfloat16): more heads
    # than a tile's 16, a latent of more than one chunk of 128 value columns, and one of a single 16
    "wide_latent": config([latent_layer(20, 16, 16, 16, 160, dense(64)), mingru_layer(48, None),
                           latent_layer(6, 32, 32, 24, 64, dense(48)), latent_layer(3, 8, 16, 8, 16, None)], width=80, vocab=120),
    "experts_only": config([mingru_layer(48, moe(9, 3, 24, limit=3.0)), latent_layer(2, 16, 8, 16, 32, moe(4, 4, 40))],
                           width=56, vocab=150, softcap=4.0),
}


def weights_for(cfg: dict, seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    W: Dict[str, torch.Tensor] = {}

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=gen, dtype=torch.float32) * std + mean

    def matrix(name, out, inp, gain=1.0):
        W[name] = normal(out, inp, std=gain / math.sqrt(inp))

    W["embed"] = normal(cfg["vocab"], D, std=1.0 / math.sqrt(D))
    W["embed.norm"] = normal(D, std=0.2)
    W["final.norm"] = normal(D, std=0.2)
    for i, layer in enumerate(cfg["layers"]):
        p, m, mlp = f"l{i}", layer["mixer"], layer["mlp"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if mlp is not None else ()):
            W[f"{p}.{n}"] = normal(D, std=0.2)
        W[f"{p}.dwa"] = normal(i + 2, std=0.15, mean=0.6)
        if layer["type"] == "mingru":
            w = m["width"]
            matrix(f"{p}.mix.z", w, D, 1.5)
            matrix(f"{p}.mix.x", w, D, 1.5)
            matrix(f"{p}.mix.g", w, D)
            matrix(f"{p}.mix.o", D, w)
            W[f"{p}.mix.z.b"] = normal(w, std=1.0)
            W[f"{p}.mix.x.b"] = normal(w, std=0.5)
        else:
            H, d, r, dv, k = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            matrix(f"{p}.mix.q", H * (d + r), D, sharp / (m["scale"] * math.sqrt(d + r)))      # scores of spread `sharp`
            matrix(f"{p}.mix.dkv", k + r, D, 1.5)
            W[f"{p}.mix.dkv.norm"] = normal(k, std=0.2, mean=1.0)
            matrix(f"{p}.mix.uk", H * d, k)
            matrix(f"{p}.mix.uv", H * dv, k)
            matrix(f"{p}.mix.o", D, H * dv)
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            matrix(f"{p}.mlp.up", mlp["ff"], D)
            matrix(f"{p}.mlp.down", D, mlp["ff"])
            W[f"{p}.mlp.act"] = torch.tensor([0.7, 0.4, -0.2, 0.1]) + normal(4, std=0.05)
        else:
            matrix(f"{p}.mlp.router", mlp["router"]["experts"], D, 2.0)
            for e in range(mlp["router"]["experts"]):
                matrix(f"{p}.mlp.e{e}.gate", mlp["expert"]["ff"], D, 2.0)      # some products beyond the limit
                matrix(f"{p}.mlp.e{e}.up", mlp["expert"]["ff"], D, 2.0)
                matrix(f"{p}.mlp.e{e}.down", D, mlp["expert"]["ff"])
    return {name: t.to(torch.bfloat16).float() for name, t in W.items()}


def write_model(path: str, cfg: dict, W: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, os.path.join(path, "model.safetensors"))
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return path


def oracle(cfg: dict, W: Dict[str, torch.Tensor], requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    W64 = {k: v.double() for k, v in W.items()}
    return {rid: plain.forward(cfg, W64, toks).float() for rid, toks in requests.items()}


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per position: root mean square of the logit difference over the vocabulary, relative to that of the logits."""
    return (got.double() - want.double()).pow(2).mean(dim=1).sqrt() / want.double().pow(2).mean(dim=1).sqrt().clamp_min(1e-3)


# float32: the engine's sums against the float64 oracle. bfloat16: products of bfloat16 operands and a bfloat16 cache.
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def assert_matches(got: Dict[str, torch.Tensor], want: Dict[str, torch.Tensor], dtype, what: str, share: float = 1.0):
    """Every position of every request within the type's tolerance; ``share`` < 1 allows that share of positions only
    (bfloat16 with routed experts: a router's close call may fall the other way than in float64)."""
    tol = TOL[dtype]
    bad, total, worst = [], 0, 0.0
    for rid, ref in want.items():
        assert got[rid].shape == ref.shape, f"{what}: request {rid} has shape {tuple(got[rid].shape)}, expected {tuple(ref.shape)}"
        err = row_errors(got[rid], ref)
        total += err.numel()
        worst = max(worst, float(err.max()))
        bad += [(rid, int(i), float(err[i])) for i in (err > tol).nonzero().flatten()]
    assert len(bad) <= (1.0 - share) * total, (f"{what}: {len(bad)} of {total} positions are further than {tol:.0e} from the plain "
                                               f"implementation (worst {worst:.2e}); the first: {bad[:5]}")
