"""Token embedding (src/llm_pipeline/models/qwen3/custom_builder.py:300-305,323: a plain row
gather) and the output head (:387-391,415: a bias-free linear layer whose weight is the embedding
table when ``tie_word_embeddings`` is set). The head returns float32 logits."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .base import Embedding, Head, TensorGetter
from .registry import register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, name: Optional[str] = None, scale: float = 1.0):
        """``name``: the table's full tensor name where it is not ``<prefix>.weight``; ``scale``: a factor on every row."""
        self.prefix, self.vocab_size, self.hidden_size = prefix, int(vocab_size), int(hidden_size)
        self.scale = float(scale)
        self.name = name or f"{prefix}.weight"
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(self.name, "matrix").contiguous()

    def forward(self, ctx) -> torch.Tensor:
        out = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=ctx.device)
        kernels.embedding(ctx.token_ids, self.weight, out, self.scale)
        return out


@register_embedding("normed_token_embedding")
class NormedTokenEmbedding(TokenEmbedding):
    """A row gather followed by an RMS norm of the row with a weight of its own (``offset + w``), in one kernel."""

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, eps: float, offset: float = 0.0,
                 name: Optional[str] = None, norm_name: Optional[str] = None):
        super().__init__(prefix, vocab_size, hidden_size, name)
        self.eps, self.offset = float(eps), float(offset)
        self.norm_name = norm_name or f"{prefix}.norm.weight"
        self.norm_weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = super().param_specs()
        specs[self.norm_name] = ParamSpec((self.hidden_size,), role="vector", init="small" if self.offset else "norm")
        return specs

    def load(self, get: TensorGetter) -> None:
        super().load(get)
        self.norm_weight = (get(self.norm_name, "vector").float() + self.offset).contiguous()

    def forward(self, ctx) -> torch.Tensor:
        out = torch.empty((ctx.num_tokens, self.hidden_size), dtype=torch.float32, device=ctx.device)
        kernels.embedding_norm(ctx.token_ids, self.weight, self.norm_weight, 0.0, self.eps, out)
        return out


@register_head("linear_head")
class LinearHead(Head):
    graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None,
                 tied_name: Optional[str] = None, softcap: Optional[float] = None, name: Optional[str] = None):
        """``tied_to``: the prefix of the embedding whose table the head uses (``tied_name``: that table's full tensor
        name where it is not ``<tied_to>.weight``). ``softcap``: logits become ``cap * tanh(logits / cap)``. ``name``: the
        full name of an untied head's matrix where it is not ``<prefix>.weight``."""
        self.name = name or f"{prefix}.weight"
        self.prefix, self.vocab_size, self.hidden_size, self.tied_to = prefix, int(vocab_size), int(hidden_size), tied_to
        self.tied_name = tied_name or (f"{tied_to}.weight" if tied_to else None)
        self.softcap = float(softcap) if softcap else None
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        # A tied head has no tensor of its own; a checkpoint may still carry a copy, which must be one.
        return {self.name: ParamSpec((self.vocab_size, self.hidden_size), optional=self.tied_to is not None)}

    def copies(self) -> Dict[str, str]:
        # The reference makes the head's parameter the embedding's own tensor when tie_word_embeddings is set
        # (models/qwen3/custom_builder.py:389-391), so a checkpoint it wrote holds the same values under both names.
        return {self.name: self.tied_name} if self.tied_to else {}

    def load(self, get: TensorGetter) -> None:
        self.weight = get(self.tied_name if self.tied_to else self.name, "matrix")

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        logits = linear(x, self.weight, out_dtype=torch.float32)
        if self.softcap is not None:
            kernels.softcap(logits, self.softcap)
        return logits
