"""Small Razelorn configurations with weights made for the tests, and the comparison with the plain implementation.

The weights are drawn so that every mechanism carries weight in the logits (projections of unit gain, norm weights and
biases well away from their neutral values, a factor between the two attention maps far from zero, a router correction
that changes choices) and are rounded to bfloat16 once, so the engine in either type and the float64 oracle read the
same numbers. ``sharp`` is the spread of the attention scores (queries and keys are normed, so the score scale alone
sets it): at 6 a softmax puts most of its weight on one or two keys, wherever they are, and a key that is lost, shifted
by one, read from the wrong page or wrongly inside a window changes the result by its whole value.
"""

from __future__ import annotations

import copy
import json
import math
import os
from typing import Dict, List, Optional

import torch

import plain_razelorn as plain

SCALING = {"factor": 4.0, "low": 1.0, "high": 8.0, "original": 64}      # wavelengths of 8 to 64 positions are blended


def attention(heads: int, kv_heads: int, dim: int, vdim: int, mlp, window: Optional[int] = None, rot_dims: Optional[int] = None,
              base: float = 10000.0, scaling: Optional[dict] = None, diff: float = 0.4, sharp: float = 1.0, weights_of: Optional[int] = None) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": sharp / math.sqrt(dim), "diff": diff}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mixer["rot"]["scaling"] = dict(scaling)
    layer = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        layer["weights_of"] = weights_of
    return layer


def again(layers: List[dict], j: int) -> dict:
    """A layer that uses layer j's tensors."""
    layer = copy.deepcopy(layers[j])
    layer["weights_of"] = j
    return layer


def dense(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def moe(experts: int, top: int, ff: int, identity: int = 0, shared: Optional[int] = None) -> dict:
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def config(layers: List[dict], width: int = 80, vocab: int = 211, eps: float = 1e-5, scale: float = 2.0) -> dict:
    return {"architecture": "Razelorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


def _mixed() -> dict:
    layers = [attention(6, 2, 32, 48, moe(7, 2, 40, identity=2, shared=56), window=24, rot_dims=16, scaling=SCALING),
              attention(4, 4, 16, 16, dense(96), window=None, rot_dims=16, diff=0.25)]
    layers.append(again(layers, 0))
    layers.append(attention(3, 1, 64, 32, None, window=50, rot_dims=8, base=500.0, diff=0.6))
    layers.append(again(layers, 1))
    return config(layers)


def _shared_weights() -> dict:
    layers = [attention(8, 2, 16, 32, dense(72), window=17, rot_dims=8, scaling=SCALING, diff=0.3)]
    layers += [again(layers, 0), again(layers, 0)]
    layers.append(attention(2, 2, 48, 96, moe(5, 5, 24, identity=0, shared=None), window=33, rot_dims=48))
    return config(layers, width=64, vocab=130, eps=3e-6, scale=0.5)


# Several shapes: key/value heads that are one, several or as many as the query heads; values wider than, as wide as and
# narrower than keys; windows shorter and longer than a page, and none; a rotation of all, part and none of a key, with
# and without frequency rescaling; layers without a feed-forward; routers with and without identity experts and shared
# expert, one choice per token and all of them; layers that use an earlier layer's tensors once and twice; sizes that
# are no multiples of 16 (the general kernels also in bfloat16); widths that are no multiples of 4.
CONFIGS: Dict[str, dict] = {
    "mixed": _mixed(),
    "shared_weights": _shared_weights(),
    "odd_sizes": config([attention(3, 3, 12, 20, moe(3, 1, 30, identity=1, shared=18), window=9, rot_dims=6, scaling=SCALING),
                         attention(5, 1, 24, 8, dense(50), window=None, rot_dims=None),
                         attention(2, 1, 40, 40, None, window=70, rot_dims=40, base=100.0)], width=54, vocab=97, scale=1.0),
    "no_window": config([attention(4, 2, 32, 64, dense(64), window=None, rot_dims=32, scaling=SCALING),
                         attention(4, 1, 16, 32, moe(6, 3, 32, identity=3, shared=32), window=None, rot_dims=8)], width=64, vocab=120),
    "wide_heads": config([attention(2, 1, 128, 128, dense(64), window=40, rot_dims=64),
                          attention(32, 2, 16, 16, None, window=100, rot_dims=16, scaling=SCALING)], width=96, vocab=150),
}


def sharpen(cfg: dict, sharp: float) -> dict:
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] = sharp / math.sqrt(layer["mixer"]["dim"])
    return cfg


def weights_for(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    W: Dict[str, torch.Tensor] = {}

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(*shape, generator=gen, dtype=torch.float32) * std + mean

    def matrix(name, out, inp, gain=1.0):
        W[name] = normal(out, inp, std=gain / math.sqrt(inp))

    W["embed"] = normal(cfg["vocab"], D, std=1.0)
    W["head"] = normal(cfg["vocab"], D, std=1.0 / math.sqrt(D))
    W["final.norm"], W["final.norm.b"] = normal(D, std=0.2, mean=1.0), normal(D, std=0.2)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m, mlp = f"l{i}", layer["mixer"], layer["mlp"]
        W[f"{p}.norm1"], W[f"{p}.norm1.b"] = normal(D, std=0.2, mean=1.0), normal(D, std=0.2)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        matrix(f"{p}.mix.q", H * 2 * d, D)
        matrix(f"{p}.mix.k", G * 2 * d, D)
        matrix(f"{p}.mix.v", G * dv, D, 1.5)
        matrix(f"{p}.mix.o", D, H * dv)
        W[f"{p}.mix.q.norm"], W[f"{p}.mix.k.norm"] = normal(d, std=0.2, mean=1.0), normal(d, std=0.2, mean=1.0)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            W[f"{p}.mix.{n}"] = normal(d, std=0.9 / d ** 0.25)            # exp(lq . lk) of spread about 0.8
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            matrix(f"{p}.mlp.up", mlp["ff"], D, 1.4)
            matrix(f"{p}.mlp.down", D, mlp["ff"])
        else:
            outputs = mlp["router"]["experts"] + mlp["router"].get("identity", 0)
            matrix(f"{p}.mlp.router", outputs, D, 1.5)
            W[f"{p}.mlp.correction"] = normal(outputs, std=0.5 / outputs)
            for e in range(mlp["router"]["experts"]):
                matrix(f"{p}.mlp.e{e}.gate", mlp["expert"]["ff"], D, 2.0)
                matrix(f"{p}.mlp.e{e}.up", mlp["expert"]["ff"], D, 2.0)
                matrix(f"{p}.mlp.e{e}.down", D, mlp["expert"]["ff"], 2.0)
            if mlp.get("shared"):
                matrix(f"{p}.mlp.shared.gate", mlp["shared"]["ff"], D, 2.0)
                matrix(f"{p}.mlp.shared.up", mlp["shared"]["ff"], D, 2.0)
                matrix(f"{p}.mlp.shared.down", D, mlp["shared"]["ff"])
                matrix(f"{p}.mlp.shared.sg", 1, D, 2.0)
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
