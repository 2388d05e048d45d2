"""Causal attention whose cache holds one small latent vector per token instead of keys and values per head.

With h the mixer's input, H heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key entries, values of
``vdim`` and a latent of ``kv_rank`` entries::

    q = Wq h                                  per head [dim | rot_dim]; the rot_dim part is rotated by the position
    [l | k_r] = Wdkv h                        kv_rank + rot_dim entries
    c = rms_norm(l) * w_c                     the latent; k_r is rotated by the position and shared by all heads
    k_h = Wuk_h c,  v_h = Wuv_h c             never formed: see below
    score_h(i, j) = (q_h,plain(i) . k_h(j) + q_h,rot(i) . k_r(j)) * scale,  j <= i,  softmax over j
    out = Wo concat_h(sum_j p_h(i, j) v_h(j))

Only ``[c | k_r]`` is cached (``TokenPagesSpec``: one row of kv_rank + rot_dim entries per token). Both up-projections
are linear, so they move to the query's side: ``q_h,plain . (Wuk_h c) = (Wuk_h^T q_h,plain) . c`` and
``sum_j p_j (Wuv_h c_j) = Wuv_h (sum_j p_j c_j)``. Every head then attends over the same cached rows, with a query of
kv_rank + rot_dim entries and the rows' first kv_rank entries as values, in prompts and in decoding alike; the two maps
are one batched product over the heads before and after the attention kernel. Scores, softmax, norm and angles are
float32. ``rot_dims`` (<= rot_dim) entries of the rotated parts take the rotation, the rest pass unchanged."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.spec import TokenPagesSpec
from ..ops import kernels
from ..ops.linear import batched_linear, linear
from ..weights.source import ParamSpec
from .attention import AttentionPolicy
from .base import LayerCache, Mixer, TensorGetter
from .registry import register_mixer


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True      # a step only writes this step's cache rows: repeating it changes nothing

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, norm_eps: float, position: Optional[str] = None, rot_dims: Optional[int] = None):
        self.prefix, self.hidden_size, self.num_heads = prefix, int(hidden_size), int(num_heads)
        self.dim, self.rot_dim, self.vdim, self.kv_rank = int(dim), int(rot_dim), int(vdim), int(kv_rank)
        self.scale, self.norm_eps, self.position = float(scale), float(norm_eps), position
        self.rot_dims = (self.rot_dim if rot_dims is None else int(rot_dims)) if position else 0
        if self.rot_dims > self.rot_dim or self.rot_dims % 2:
            raise ValueError(f"{self.rot_dims} rotated entries do not fit a rotated part of {self.rot_dim}")
        if self.kv_rank > 1024:
            raise ValueError(f"the latent attention kernels take latents of at most 1024 entries, got {self.kv_rank}")
        self.q_size = self.num_heads * (self.dim + self.rot_dim)
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_norm = None

    def cache_spec(self) -> TokenPagesSpec:
        return TokenPagesSpec((self.kv_rank + self.rot_dim,), None)

    def graph_key_group(self):
        return ("latent_attention", self.num_heads, self.kv_rank, self.rot_dim)

    def param_specs(self) -> Dict[str, ParamSpec]:
        p, Hd, H = self.prefix, self.hidden_size, self.num_heads
        return {f"{p}.q": ParamSpec((self.q_size, Hd)), f"{p}.dkv": ParamSpec((self.kv_rank + self.rot_dim, Hd)),
                f"{p}.dkv.norm": ParamSpec((self.kv_rank,), role="vector", init="norm"),
                f"{p}.uk": ParamSpec((H * self.dim, self.kv_rank)), f"{p}.uv": ParamSpec((H * self.vdim, self.kv_rank)),
                f"{p}.o": ParamSpec((Hd, H * self.vdim))}

    def load(self, get: TensorGetter) -> None:
        p, H = self.prefix, self.num_heads
        self.w_in = torch.cat([get(f"{p}.q", "matrix"), get(f"{p}.dkv", "matrix")], dim=0).contiguous()
        self.c_norm = get(f"{p}.dkv.norm", "vector").contiguous()
        # per head: Wuk_h^T [kv_rank, dim] (the map of the query into the latent space) and Wuv_h [vdim, kv_rank]
        self.w_uk_t = get(f"{p}.uk", "matrix").view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = get(f"{p}.uv", "matrix").view(H, self.vdim, self.kv_rank).contiguous()
        self.w_o = get(f"{p}.o", "matrix").contiguous()

    # Blocks per SM below which a step's tiles are too few and the keys are cut into segments with blocks of their own
    # (decode steps, short portions over long contexts); and the context from which that is worth a second kernel.
    SEGMENTS_BELOW_BLOCKS_PER_SM = 2.0
    SEGMENTS_MIN_CONTEXT = 2 * kernels.LATENT_SEGMENT_KEYS

    def attend(self, ctx, q_lat, q_rot, out, cache: LayerCache) -> None:
        """Attention of the step's rows over the cache: the tensor-core kernel for bfloat16 where it serves the sizes,
        else the general kernel (float32, sizes that are no multiples of 16)."""
        tables = ctx.block_tables[cache.group]
        if not kernels.latent_mma_supports(q_lat.dtype, self.kv_rank, self.rot_dim, cache.pages.shape[1]) or self.dim % 8 or self.rot_dim % 8:
            kernels.latent_attention(q_lat, q_rot, cache.pages, tables, ctx.token_request, ctx.positions, out, self.scale)
            return
        per_tile = kernels.latent_mma_tokens_per_tile(self.num_heads)
        key = ("latent_attention_tiles", per_tile)
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
        longest = ctx.decode_ctx_bound or ctx.max_ctx_len
        blocks = tiles[0].numel() * -(-self.num_heads // 16) * -(-self.kv_rank // 128)
        segments = 0
        if blocks < self.SEGMENTS_BELOW_BLOCKS_PER_SM * kernels.sm_count() and longest >= self.SEGMENTS_MIN_CONTEXT:
            segments = -(-longest // kernels.LATENT_SEGMENT_KEYS)
        kernels.latent_attention_mma(q_lat, q_rot, cache.pages, tables, ctx.q_start, ctx.ctx_len, ctx.positions, tiles[0], tiles[1],
                                     out, self.scale, segments)

    def forward(self, x, ctx, cache: LayerCache):
        if cache.pages is None or cache.group is None:
            raise RuntimeError("the latent attention mixer needs the pages of its cache")
        N, H, rank, rot = ctx.num_tokens, self.num_heads, self.kv_rank, self.rot_dim
        qd = linear(x, self.w_in)                                        # [N, H (dim + rot) | rank + rot]
        cos = sin = None
        if self.rot_dims:
            cos, sin = ctx.position_tables[self.position]
        kernels.latent_kv_post(qd, H, self.dim, rot, rank, self.c_norm, self.norm_eps, cos, sin, self.rot_dims,
                               ctx.slot_mapping[cache.group] if cache.writes else None, cache.pages if cache.writes else None)
        q = qd[:, :self.q_size].view(N, H, self.dim + rot)
        q_lat = torch.empty((N, H, rank), dtype=x.dtype, device=x.device)
        batched_linear(q[:, :, :self.dim].transpose(0, 1), self.w_uk_t, q_lat.transpose(0, 1))
        mixed = torch.empty((N, H, rank), dtype=x.dtype, device=x.device)
        self.attend(ctx, q_lat, q[:, :, self.dim:], mixed, cache)
        values = torch.empty((N, H, self.vdim), dtype=x.dtype, device=x.device)
        batched_linear(mixed.transpose(0, 1), self.w_uv, values.transpose(0, 1))
        return linear(values.view(N, H * self.vdim), self.w_o, out_dtype=torch.float32), None
