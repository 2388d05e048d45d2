"""Differential attention over the paged cache, as a mixer.

With h the mixer's input, H query heads, G key/value heads (query head i uses key/value head i // (H / G)), keys and
queries of ``dim`` entries, values of ``vdim``::

    q = Wq h   [H, 2, dim]      two queries per head (map 1, map 2)
    k = Wk h   [G, 2, dim]      two keys per key/value head
    v = Wv h   [G, vdim]        one value, shared by both maps
    q, k <- rms_norm over dim with one weight for all of q and one for all of k, then rotation of the first
            ``rotary_dim`` entries (entry i with entry i + rotary_dim / 2)
    a_m(i) = sum_j softmax_j(q_m(i) . k_m(j) * scale) v(j)      m = 1, 2; j <= i, and i - j < window if there is one
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff             one number per layer, taken once at load time in float32
    o(i) = rms_norm(a_1(i) - lambda a_2(i)) * (1 - diff)        per head over its vdim entries, no weight
    out = Wo concat_heads(o)

The three projections are one product against [Wq; Wk; Wv]; one kernel norms and rotates q and k and writes a cache row
[k_1 | k_2 | v] per key/value head and token (``HeadRowPagesSpec``); the attention kernel reads all keys and values from
the pages, this step's included, and leaves the finished o: both softmaxes, the difference and its norm happen inside it.
Scores, softmaxes, the difference and the norms are float32. bfloat16 steps take the tensor-core kernel where it serves
the sizes (decoding over long contexts with the keys cut into segments), float32 steps and other sizes the general one."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import HeadRowPagesSpec
from ..ops import kernels
from ..ops.linear import linear
from ..weights.source import ParamSpec
from .attention import AttentionPolicy
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True      # a step only writes this step's cache rows: repeating it changes nothing

    # Blocks per SM below which a step's tiles are too few and the keys are cut into segments with blocks of their own
    # (decode steps, short portions over long contexts); and the keys a request must see for that to be worth a second kernel.
    SEGMENTS_BELOW_BLOCKS_PER_SM = 1.0
    SEGMENTS_MIN_CONTEXT = 2 * kernels.DIFF_SEGMENT_KEYS

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float,
                 diff: float, norm_eps: float, window: Optional[int] = None, position: Optional[str] = None,
                 rotary_dim: int = 0, names: Optional[Dict[str, str]] = None):
        """``names``: the tensors' names below ``prefix`` where they are not q, k, v, o, q.norm, k.norm, lq1, lk1, lq2, lk2."""
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
        if not 0 < dim <= 256:
            raise ValueError(f"the differential attention kernels take key sizes up to 256, got {dim}")
        if not 0 < vdim <= 512:
            raise ValueError(f"the differential attention kernels take value sizes up to 512, got {vdim}")
        self.prefix, self.hidden_size = prefix, int(hidden_size)
        self.num_heads, self.num_kv_heads, self.dim, self.vdim = int(num_heads), int(num_kv_heads), int(dim), int(vdim)
        self.scale, self.diff, self.norm_eps = float(scale), float(diff), float(norm_eps)
        self.window = int(window) if window else None
        self.position = position
        self.rotary_dim = int(rotary_dim) if position else 0
        if self.rotary_dim > self.dim or self.rotary_dim % 2:
            raise ValueError(f"{self.rotary_dim} rotated entries do not fit keys of {self.dim}")
        self.q_size, self.k_size, self.v_size = 2 * self.num_heads * self.dim, 2 * self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim
        self.names = {n: n for n in ("q", "k", "v", "o", "q.norm", "k.norm", "lq1", "lk1", "lq2", "lk2")}
        self.names.update(names or {})
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None
        self.lam = 0.0

    def cache_spec(self) -> HeadRowPagesSpec:
        return HeadRowPagesSpec(self.num_kv_heads, 2 * self.dim + self.vdim, self.window)

    def graph_key_group(self):
        return ("differential_attention", self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.window)

    def _name(self, key: str) -> str:
        return f"{self.prefix}.{self.names[key]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        Hd = self.hidden_size
        specs = {self._name("q"): ParamSpec((self.q_size, Hd)), self._name("k"): ParamSpec((self.k_size, Hd)),
                 self._name("v"): ParamSpec((self.v_size, Hd)), self._name("o"): ParamSpec((Hd, self.num_heads * self.vdim)),
                 self._name("q.norm"): ParamSpec((self.dim,), role="vector", init="norm"),
                 self._name("k.norm"): ParamSpec((self.dim,), role="vector", init="norm")}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            specs[self._name(n)] = ParamSpec((self.dim,), role="vector", init="normal")
        return specs

    def load(self, get: TensorGetter) -> None:
        self.w_qkv = torch.cat([get(self._name(n), "matrix") for n in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = get(self._name("o"), "matrix").contiguous()
        self.q_norm = get(self._name("q.norm"), "vector").contiguous()
        self.k_norm = get(self._name("k.norm"), "vector").contiguous()
        if self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        l = {n: get(self._name(n), "vector").float() for n in ("lq1", "lk1", "lq2", "lk2")}
        lam = torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum()) + self.diff     # float32
        self.lam = float(lam.item())

    def _tiles(self, ctx, per_tile: int):
        key = ("differential_attention_tiles", per_tile)
        tiles = ctx.memo.get(key)
        if tiles is None:
            if ctx.max_q_len == 1:
                # one token a request: tile r is request r (made on the device, so that a captured step holds no copy from the host)
                tiles = (torch.arange(ctx.num_requests, dtype=torch.int32, device=ctx.device),
                         torch.zeros(ctx.num_requests, dtype=torch.int32, device=ctx.device))
            else:
                req, tok0, _seg, _slot, _places = AttentionPolicy.plan_items(ctx.starts, ctx.q_lens, per_tile, 0, 1, 1, kernels.sm_count())
                host = torch.tensor([req, tok0], dtype=torch.int32).pin_memory()
                dev = host.to(ctx.device, non_blocking=True)
                tiles = (dev[0].contiguous(), dev[1].contiguous())
            ctx.memo[key] = tiles
        return tiles

    def attend(self, ctx, qkv: torch.Tensor, out: torch.Tensor, cache: LayerCache) -> None:
        """The finished heads ``out`` [tokens, heads vdim] of the step's query rows (the first columns of ``qkv``) over the
        pages of ``cache``."""
        tables = ctx.block_tables[cache.group]
        args = (self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.window or 0, self.scale, self.lam, self.norm_eps,
                1.0 - self.diff)
        if not kernels.diff_mma_supports(qkv.dtype, self.dim, self.vdim, cache.pages.shape[2]) or qkv.stride(0) % 8:
            kernels.diff_attention(qkv, cache.pages, tables, ctx.token_request, ctx.positions, out, *args)
            return
        tile_req, tile_tok0 = self._tiles(ctx, kernels.diff_mma_tokens_per_tile(self.num_heads, self.num_kv_heads))
        longest = ctx.decode_ctx_bound or ctx.max_ctx_len
        reach = min(longest, self.window + ctx.max_q_len) if self.window else longest       # keys a tile walks at most
        blocks = tile_req.numel() * self.num_kv_heads * -(-(self.num_heads // self.num_kv_heads) // 16)
        segments = 0
        if blocks < self.SEGMENTS_BELOW_BLOCKS_PER_SM * kernels.sm_count() and reach >= self.SEGMENTS_MIN_CONTEXT:
            segments = -(-longest // kernels.DIFF_SEGMENT_KEYS)
        kernels.diff_attention_mma(qkv, cache.pages, tables, ctx.q_start, ctx.ctx_len, ctx.positions, tile_req, tile_tok0, out, *args,
                                   segments=segments, split=ctx.max_q_len == 1)

    def forward(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the differential attention mixer needs the pages of its cache")
        qkv = linear(x, self.w_qkv)
        cos = sin = None
        if self.rotary_dim:
            cos, sin = ctx.position_tables[self.position]
        kernels.diff_qkv_post(qkv, self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.q_norm, self.k_norm, self.norm_eps,
                              cos, sin, self.rotary_dim, ctx.slot_mapping[cache.group] if cache.writes else None,
                              cache.pages if cache.writes else None)
        out = torch.empty((ctx.num_tokens, self.num_heads * self.vdim), dtype=x.dtype, device=x.device)
        self.attend(ctx, qkv, out, cache)
        return linear(out, self.w_o, out_dtype=torch.float32), None
