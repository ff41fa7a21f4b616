"""A model assembled from a spec: embedding, runs of blocks, final norm, head.

Reference: ``Transformer.__init__`` and ``forward``
(torchllms/models/networks.py:790-810, :1017-1047): embed, run every block,
keep the wanted rows, final norm, output projection (tied to the embedding
table when the configuration says so, :806-809).  The class knows nothing of
any architecture: the spec decides which parts exist, with which numbers, and
in which order they run.
"""

from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..parts import attention, block, ffn, norm, rope  # noqa: F401  (register the built-in parts)
from ..parts.base import BLOCKS, NORMS, BuildEnv, CacheNeed, Residual, StateNeed, as_compute
from ..parts.spec import ModelSpec
from ..weights.loader import ExpectedTensor


class Model:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device, ops, max_positions: Optional[int] = None):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.ops = ops
        self.max_positions = int(max_positions or spec.max_positions)
        self.env = BuildEnv(dim=spec.dim, dtype=dtype, device=self.device,
                            max_positions=self.max_positions, ops=ops)
        self.blocks = [BLOCKS.build(layer.block, self.env) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, self.env)
        self.graph_safe = self.final_norm.graph_safe and all(b.graph_safe for b in self.blocks)
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ----------------------------------------------------------------- weights
    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        spec = self.spec
        out: Dict[str, ExpectedTensor] = {spec.embedding_tensor: ExpectedTensor((spec.vocab_size, spec.dim))}
        for layer, blk in zip(spec.layers, self.blocks):
            for name, e in blk.expected_tensors().items():
                out[f"{layer.name}.{name}"] = e
        for name, e in self.final_norm.expected_tensors().items():
            out[f"{spec.final_norm_prefix}.{name}"] = e
        if not spec.tie_head:
            out[spec.head_tensor] = ExpectedTensor((spec.vocab_size, spec.dim))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """``tensors`` holds exactly :meth:`expected_tensors` (checked by the caller)."""
        spec = self.spec
        self.embedding = as_compute(tensors[spec.embedding_tensor], self.env)
        for layer, blk in zip(spec.layers, self.blocks):
            blk.load({name: tensors[f"{layer.name}.{name}"] for name in blk.expected_tensors()})
        self.final_norm.load({name: tensors[f"{spec.final_norm_prefix}.{name}"]
                              for name in self.final_norm.expected_tensors()})
        self.head = self.embedding if spec.tie_head else as_compute(tensors[spec.head_tensor], self.env)

    def weight_bytes(self) -> int:
        """Bytes of weights a step has to read: every layer's matrices and the head once
        (of the embedding table a step reads only the rows of its tokens)."""
        return sum(blk.weight_bytes() for blk in self.blocks) + self.final_norm.weight_bytes() \
            + self.head.numel() * self.head.element_size()

    # ------------------------------------------------------------------- cache
    def run_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]]:
        """What each run of the run order wants from the cache manager."""
        return [(self.blocks[run.layer].cache_need(), self.blocks[run.layer].state_need(), run.cache_of)
                for run in self.spec.run_order]

    # ----------------------------------------------------------------- forward
    def forward(self, ctx, views: Sequence) -> Optional[torch.Tensor]:
        """Run the step's tokens; returns float32 logits ``[n_wanted, vocab]`` or ``None``."""
        h = self.ops.embed(ctx.token_ids, self.embedding)
        residual = Residual(h)
        for i, run in enumerate(self.spec.run_order):
            self.blocks[run.layer].forward(residual, ctx, views[i])
        if ctx.n_want == 0:
            return None
        x = self.final_norm.forward(residual, rows=ctx.want_rows)
        return self.ops.linear(x, self.head, out_dtype=torch.float32)
