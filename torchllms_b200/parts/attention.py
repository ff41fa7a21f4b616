"""Grouped-query attention over the paged cache.

Reference: ``Attention`` (torchllms/models/networks.py:460-558): projections
``wq, wk, wv`` (``nn.Linear`` layout ``[out, in]``, no bias), rotary encoding of
q and k, append of k and v to the pool, attention of every query over the keys
at positions ``<=`` its own with scale ``head_dim ** -0.5`` (:842; eager form
:355-397, query head ``h`` reads kv head ``h // (H / KV)``), then ``wo``.  The
reference calls a library for the paged attention
(torchllms/models/paged_attention.py:217-301); the kernel here is our own and
treats prompt portions and single decoded tokens alike.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import (POSITION_ENCODINGS, BuildEnv, CacheNeed, Mixer, as_compute, register_mixer)
from .spec import PartSpec


@register_mixer("attention")
class PagedAttention(Mixer):
    def __init__(self, env: BuildEnv, *, dim: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, position: PartSpec, window: Optional[int] = None):
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"n_heads ({n_heads}) must be a multiple of n_kv_heads ({n_kv_heads})")
        self.env = env
        self.dim, self.n_heads, self.n_kv_heads, self.head_dim = int(dim), int(n_heads), int(n_kv_heads), int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.position = POSITION_ENCODINGS.build(position, env)
        self.graph_safe = self.position.graph_safe
        # x only goes into the q/k/v product, whose result the position encoding's kernel may scale
        self.takes_row_scaled = self.position.takes_row_scaled
        env.ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim, env.dtype)
        self.wqkv: Optional[torch.Tensor] = None
        self.wo: Optional[torch.Tensor] = None

    def cache_need(self) -> CacheNeed:
        if self.window is None:
            return CacheNeed("full", self.n_kv_heads, self.head_dim)
        return CacheNeed("window", self.n_kv_heads, self.head_dim, self.window)

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        q, kv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = {
            "wq.weight": ExpectedTensor((q, self.dim)),
            "wk.weight": ExpectedTensor((kv, self.dim)),
            "wv.weight": ExpectedTensor((kv, self.dim)),
            "wo.weight": ExpectedTensor((self.dim, q)),
        }
        # a position encoding with tensors of its own (none for rope) keeps them under "position."
        for name, e in self.position.expected_tensors().items():
            out[f"position.{name}"] = e
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # One projection for q, k and v: rows [wq; wk; wv].
        self.wqkv = torch.cat([as_compute(tensors[n], self.env) for n in ("wq.weight", "wk.weight", "wv.weight")])
        self.wo = as_compute(tensors["wo.weight"], self.env)
        self.position.load({name: tensors[f"position.{name}"] for name in self.position.expected_tensors()})

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        ops = self.env.ops
        qkv = ops.linear(x, self.wqkv, partials_ok=True)   # the encoding adds up split-K partial sums
        q = self.position.encode_and_store(qkv, ctx, cache, self.n_heads, self.n_kv_heads, self.head_dim)
        common = dict(scale=self.scale, window=self.window, page_size=cache.page_size)
        nd, B = getattr(ctx, "n_decode", 0), ctx.n_seqs
        if 0 < nd < B and ctx.max_q_len > 1:
            # decoded tokens beside prompt portions: the requests at the head of the batch bring one
            # token each and long histories, the rest bring portions; each kind goes to the kernel
            # shape made for it, both writing into one output
            o = torch.empty_like(q)
            ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table[:nd], ctx.q_start[:nd + 1],
                                ctx.kv_len[:nd], n_seqs=nd, max_q_len=1, max_kv_len=ctx.decode_kv_bound,
                                n_tokens=nd, out=o, **common)
            ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table[nd:], ctx.q_start[nd:],
                                ctx.kv_len[nd:], n_seqs=B - nd, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len,
                                out=o, allow_split=False, **common)   # (a merge pass would run over the first call's rows too)
        else:
            o = ops.paged_attention(
                q, cache.k_pages, cache.v_pages, cache.block_table, ctx.q_start, ctx.kv_len,
                n_seqs=B, max_q_len=ctx.max_q_len, max_kv_len=ctx.max_kv_len, **common)
        # the output projection is left to the norm that follows: it may add the product to the
        # residual stream in the product's own kernel, or take it and add up its partial sums
        return PendingProduct(o.view(o.shape[0], self.n_heads * self.head_dim), self.wo)
