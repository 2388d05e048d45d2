"""Typed configuration of the Zupilorn decoder, read from its ``config.json``.

A small hybrid decoder: every layer names its mixer (``type``: ``mingru``, a gated recurrence with a fixed-size state,
or ``latent_attention``, causal attention over one cached latent vector per token) and its feed-forward (``mlp``:
``dense`` with the PolyNorm activation, ``moe`` with routed experts, or null for none). Every sublayer has a norm
before and after it, all norms keep their weight around zero (the factor is 1 + w), the embedding has a norm of its
own, every layer hands on a learned weighted sum of all results so far, the head is the embedding table, and the
logits pass a tanh soft cap. Keys::

    {"architecture": "Zupilorn", "vocab": V, "width": D, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "mingru", "mixer": {"width": W}, "mlp": {"kind": "dense", "ff": F}},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "kv_rank": k, "scale": s,
                           "rot": {"base": b, "dims": n}},
                 "mlp": {"kind": "moe", "expert": {"ff": F, "limit": l}, "router": {"experts": E, "top": t}}},
                {..., "mlp": null}]}

Tensor names: ``embed``, ``embed.norm``, ``final.norm``; per layer i ``l<i>.norm1``, ``.norm1b`` (around the mixer),
``.norm2``, ``.norm2b`` (around the feed-forward), ``.dwa`` (the i + 2 depth weights), ``.mix.*`` and ``.mlp.*``."""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from .base import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

_MIXERS = ("mingru", "latent_attention")
_MLPS = ("dense", "moe")


@dataclass(frozen=True)
class ZupilornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: Optional[float]
    layers: Tuple[Dict[str, Any], ...] = field(default_factory=tuple)
    max_position_embeddings: int = 1 << 20

    architecture = "Zupilorn"
    model_type = "zupilorn"

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
    def from_json(cls, data: Dict[str, Any]) -> "ZupilornConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if data.get(k) is None]
        if missing:
            raise ValueError(f"Zupilorn config.json lacks required keys: {missing}")
        if "eps" not in data["norm"]:
            raise ValueError("Zupilorn config.json lacks norm.eps")
        cap = data.get("logit_softcap")
        config = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                     logit_softcap=float(cap) if cap else None, layers=tuple(copy.deepcopy(list(data["layers"]))),
                     max_position_embeddings=int(data.get("max_position_embeddings", 1 << 20)))
        config.validate()
        return config

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
            needs = ("width",) if kind == "mingru" else ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale")
            lacking = [k for k in needs if mixer.get(k) is None]
            if lacking:
                problems.append(f"layer {i}: the {kind} mixer lacks {lacking}")
            elif kind == "latent_attention" and mixer["rot_dim"] > 0:
                rot = mixer.get("rot") or {}
                if rot.get("base") is None:
                    problems.append(f"layer {i}: a rotated part needs rot.base")
                elif int(rot.get("dims", mixer["rot_dim"])) > int(mixer["rot_dim"]) or int(rot.get("dims", mixer["rot_dim"])) % 2:
                    problems.append(f"layer {i}: rot.dims must be even and at most rot_dim")
            if mlp is not None:
                if mlp.get("kind") not in _MLPS:
                    problems.append(f"layer {i}: unknown mlp kind {mlp.get('kind')!r} (known: {list(_MLPS)})")
                elif mlp["kind"] == "dense" and mlp.get("ff") is None:
                    problems.append(f"layer {i}: a dense mlp needs ff")
                elif mlp["kind"] == "moe":
                    expert, router = mlp.get("expert") or {}, mlp.get("router") or {}
                    if expert.get("ff") is None or expert.get("limit") is None or router.get("experts") is None or router.get("top") is None:
                        problems.append(f"layer {i}: a moe mlp needs expert.ff, expert.limit, router.experts and router.top")
                    elif not 0 < int(router["top"]) <= int(router["experts"]):
                        problems.append(f"layer {i}: router.top must lie in 1..router.experts")
        if problems:
            raise ValueError("invalid Zupilorn configuration: " + "; ".join(problems))

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
                "logit_softcap": self.logit_softcap, "layers": copy.deepcopy(list(self.layers))}

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

    def _rotary_name(self, base: float, dims: int) -> str:
        return f"rotary_{dims}_{base!r}"

    def model_spec(self) -> ModelSpec:
        D = self.width

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"size": D, "eps": self.norm_eps, "offset": 1.0, "name": name})

        positions: Dict[str, PartSpec] = {}
        layers = []
        for i, layer in enumerate(self.layers):
            p, m, mlp = f"l{i}", layer["mixer"], layer.get("mlp")
            if layer["type"] == "mingru":
                mixer = PartSpec("min_gru", {"hidden_size": D, "width": int(m["width"])}, f"{p}.mix")
            else:
                position = None
                rot_dims = 0
                if int(m["rot_dim"]) > 0:
                    rot = m["rot"]
                    rot_dims = int(rot.get("dims", m["rot_dim"]))
                    if rot_dims:
                        position = self._rotary_name(float(rot["base"]), rot_dims)
                        positions.setdefault(position, PartSpec("rotary", {"rotary_dim": rot_dims, "theta": float(rot["base"]),
                                                                           "scaling": 1.0}))
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                    "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]),
                    "norm_eps": self.norm_eps, "position": position, "rot_dims": rot_dims}, f"{p}.mix")
            norms = {"mixer": norm(f"{p}.norm1"), "mixer_out": norm(f"{p}.norm1b")}
            feed_forward = None
            if mlp is not None:
                norms.update({"feed_forward": norm(f"{p}.norm2"), "feed_forward_out": norm(f"{p}.norm2b")})
                if mlp["kind"] == "dense":
                    feed_forward = PartSpec("poly_norm_mlp", {"hidden_size": D, "intermediate_size": int(mlp["ff"]),
                                                              "eps": self.norm_eps}, f"{p}.mlp")
                else:
                    feed_forward = PartSpec("routed_experts", {
                        "hidden_size": D, "intermediate_size": int(mlp["expert"]["ff"]), "num_experts": int(mlp["router"]["experts"]),
                        "top": int(mlp["router"]["top"]), "limit": float(mlp["expert"]["limit"])}, f"{p}.mlp")
            layers.append(LayerSpec(block="sandwich_norm_residual", mixer=mixer, feed_forward=feed_forward, norms=norms,
                                    depth_mix=PartSpec("weighted_average", {"count": i + 2, "name": f"{p}.dwa"}, p)))
        spec = ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D,
            embedding=PartSpec("normed_token_embedding", {"vocab_size": self.vocab, "hidden_size": D, "eps": self.norm_eps,
                                                          "offset": 1.0, "name": "embed", "norm_name": "embed.norm"}, "embed"),
            positions=positions, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, i) for i in range(len(layers))),
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D, "tied_to": "embed", "tied_name": "embed",
                                          "softcap": self.logit_softcap}, "head"),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture("Zupilorn", ZupilornConfig)
