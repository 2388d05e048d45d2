"""Typed configuration of the Razelorn decoder, read from its ``config.json``.

A small decoder whose layers run their two sublayers side by side: with h = layer_norm(x), x += mixer(h) + mlp(h). The
mixer is differential attention (two softmax maps per head over shared values, grouped key/value heads, a norm on
queries and keys, a rotation of part of each key with wavelength-dependent frequency rescaling, a sliding window); the
feed-forward (``mlp``) is ``dense`` (squared ReLU), ``moe`` (softmax router with a correction for the choice, gated SiLU
experts, identity experts, an always-on shared expert behind a sigmoid gate) or null for none. A layer may use another
layer's tensors (``weights_of``) with a cache of its own. The embedding is scaled; final layer norm and an untied head.
Keys::

    {"architecture": "Razelorn", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": c, "diff": f, "mask": {"size": w},
                           "rot": {"base": b, "dims": n, "scaling": {"factor": .., "low": .., "high": .., "original": ..}}},
                 "mlp": {"kind": "dense", "ff": F}},
                {..., "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": t, "identity": i},
                              "shared": {"ff": S}}},
                {..., "weights_of": 1}, {..., "mlp": null}]}

Tensor names: ``embed``, ``final.norm``, ``final.norm.b``, ``head``; per layer i with tensors of its own ``l<i>.norm1``,
``l<i>.norm1.b``, ``l<i>.mix.{q,k,v,o,q.norm,k.norm,lq1,lk1,lq2,lk2}`` and ``l<i>.mlp.{up,down}`` or
``l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down,sg}}``."""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

_MIXERS = ("attention",)
_MLPS = ("dense", "moe")


@dataclass(frozen=True)
class RazelornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    layers: Tuple[Dict[str, Any], ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20

    architecture = "Razelorn"
    model_type = "razelorn"

    # the names other parts of the engine read from any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "RazelornConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if data.get(k) is None]
        if missing:
            raise ValueError(f"Razelorn config.json lacks required keys: {missing}")
        if "eps" not in data["norm"]:
            raise ValueError("Razelorn config.json lacks norm.eps")
        scale = (data.get("embedding") or {}).get("scale", 1.0)
        config = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                     embedding_scale=float(1.0 if scale is None else scale), layers=tuple(copy.deepcopy(list(data["layers"]))),
                     max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)))
        config.validate()
        return config

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it names another with ``weights_of``)."""
        j = self.layers[i].get("weights_of")
        return i if j is None else int(j)

    def validate(self) -> None:
        problems: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            problems.append(f"vocab and width must be positive, got {self.vocab} and {self.width}")
        if not self.norm_eps > 0:
            problems.append(f"norm.eps must be positive, got {self.norm_eps}")
        if not self.layers:
            problems.append("the model has no layers")
        for i, layer in enumerate(self.layers):
            kind, mixer, mlp = layer.get("type"), layer.get("mixer") or {}, layer.get("mlp")
            if kind not in _MIXERS:
                problems.append(f"layer {i}: unknown type {kind!r} (known: {list(_MIXERS)})")
                continue
            j = layer.get("weights_of")
            if j is not None:
                if not 0 <= int(j) < len(self.layers) or int(j) == i or self.layers[int(j)].get("weights_of") is not None:
                    problems.append(f"layer {i}: weights_of must name another layer that has tensors of its own, got {j}")
                    continue
                # the layer runs layer j's parts, so layer j's description is the one that counts
                kind, mixer, mlp = self.layers[int(j)].get("type"), self.layers[int(j)].get("mixer") or {}, self.layers[int(j)].get("mlp")
            lacking = [k for k in ("heads", "kv_heads", "dim", "vdim", "scale", "diff") if mixer.get(k) is None]
            if lacking:
                problems.append(f"layer {i}: the attention mixer lacks {lacking}")
            else:
                if int(mixer["heads"]) % int(mixer["kv_heads"]):
                    problems.append(f"layer {i}: {mixer['heads']} heads cannot share {mixer['kv_heads']} key/value heads")
                rot = mixer.get("rot")
                if rot and int(rot.get("dims", 0) or 0) > 0:
                    if rot.get("base") is None:
                        problems.append(f"layer {i}: a rotation needs rot.base")
                    if int(rot["dims"]) > int(mixer["dim"]) or int(rot["dims"]) % 2:
                        problems.append(f"layer {i}: rot.dims must be even and at most dim")
                    scaling = rot.get("scaling")
                    if scaling and [k for k in ("factor", "low", "high", "original") if scaling.get(k) is None]:
                        problems.append(f"layer {i}: rot.scaling needs factor, low, high and original")
                size = (mixer.get("mask") or {}).get("size")
                if size is not None and int(size) <= 0:
                    problems.append(f"layer {i}: mask.size must be positive")
            if mlp is not None:
                if mlp.get("kind") not in _MLPS:
                    problems.append(f"layer {i}: unknown mlp kind {mlp.get('kind')!r} (known: {list(_MLPS)})")
                elif mlp["kind"] == "dense" and mlp.get("ff") is None:
                    problems.append(f"layer {i}: a dense mlp needs ff")
                elif mlp["kind"] == "moe":
                    expert, router = mlp.get("expert") or {}, mlp.get("router") or {}
                    if expert.get("ff") is None or router.get("experts") is None or router.get("top") is None:
                        problems.append(f"layer {i}: a moe mlp needs expert.ff, router.experts and router.top")
                    elif not 0 < int(router["top"]) <= int(router["experts"]) + int(router.get("identity") or 0):
                        problems.append(f"layer {i}: router.top must lie in 1..router.experts + router.identity")
                    if mlp.get("shared") and mlp["shared"].get("ff") is None:
                        problems.append(f"layer {i}: a shared expert needs shared.ff")
        if problems:
            raise ValueError("invalid Razelorn configuration: " + "; ".join(problems))

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(list(self.layers))}

    def eos_token_ids(self) -> List[int]:
        return []

    def parameter_counts(self) -> Dict[str, int]:
        from ..models import expected_params

        total = 0
        for spec in expected_params(self.model_spec()).values():
            count = 1
            for n in spec.shape:
                count *= n
            total += count
        return {"total_parameters": total}

    def model_spec(self) -> ModelSpec:
        D = self.width

        def norm(name: str) -> PartSpec:
            return PartSpec("layer_norm", {"size": D, "eps": self.norm_eps, "name": name, "bias_name": f"{name}.b"})

        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        index_of: Dict[int, int] = {}                 # layer of the configuration -> its place among the layers with tensors
        for i, layer in enumerate(self.layers):
            if self.owner(i) != i:
                continue
            p, m, mlp = f"l{i}", layer["mixer"], layer.get("mlp")
            position, rot_dims = None, 0
            rot = m.get("rot")
            if rot and int(rot.get("dims", 0) or 0) > 0:
                rot_dims = int(rot["dims"])
                scaling = rot.get("scaling") or None
                rule = {k: float(scaling[k]) for k in ("factor", "low", "high", "original")} if scaling else None
                position = f"rotary_{rot_dims}_{float(rot['base'])!r}_{sorted(rule.items()) if rule else None}"
                positions.setdefault(position, PartSpec("rotary", {"rotary_dim": rot_dims, "theta": float(rot["base"]), "scaling": 1.0,
                                                                   "frequency_scaling": rule}))
            window = (m.get("mask") or {}).get("size")
            mixer = PartSpec("differential_attention", {
                "hidden_size": D, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]), "dim": int(m["dim"]),
                "vdim": int(m["vdim"]), "scale": float(m["scale"]), "diff": float(m["diff"]), "norm_eps": self.norm_eps,
                "window": int(window) if window is not None else None, "position": position, "rotary_dim": rot_dims}, f"{p}.mix")
            feed_forward = None
            if mlp is not None and mlp["kind"] == "dense":
                feed_forward = PartSpec("relu_squared_mlp", {"hidden_size": D, "intermediate_size": int(mlp["ff"])}, f"{p}.mlp")
            elif mlp is not None:
                router, shared = mlp["router"], mlp.get("shared") or None
                feed_forward = PartSpec("routed_experts", {
                    "hidden_size": D, "intermediate_size": int(mlp["expert"]["ff"]), "num_experts": int(router["experts"]),
                    "top": int(router["top"]), "score": "softmax", "form": "silu", "identity": int(router.get("identity") or 0),
                    "correction": True, "shared_size": int(shared["ff"]) if shared else None}, f"{p}.mlp")
            index_of[i] = len(layers)
            layers.append(LayerSpec(block="parallel_residual", mixer=mixer, feed_forward=feed_forward, norms={"mixer": norm(f"{p}.norm1")}))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "name": "embed",
                                                   "scale": self.embedding_scale}, "embed"),
            positions=positions, layers=tuple(layers),
            # every layer of the configuration runs once, with a cache of its own; one that uses another's tensors runs that layer's parts
            schedule=tuple(ScheduleEntry(index_of[self.owner(i)], i) for i in range(len(self.layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "name": "head"}, "head"),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture("Razelorn", RazelornConfig)
