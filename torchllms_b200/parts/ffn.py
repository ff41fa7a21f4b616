"""Dense gated feed-forward (SwiGLU).

Reference: ``FeedForward.forward`` (torchllms/models/networks.py:592-605):
``w2(silu(w1 x) * w3 x)`` with ``w1, w3: [hidden, dim]`` and ``w2: [dim, hidden]``,
no biases.  ``w1`` and ``w3`` are stacked so that one product yields gate and up.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, FeedForward, as_compute, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True
    takes_row_scaled = True      # x only goes into the gate/up product, whose activation applies the scale

    def __init__(self, env: BuildEnv, *, dim: int, hidden: int):
        self.env = env
        self.dim, self.hidden = int(dim), int(hidden)
        self.w13: Optional[torch.Tensor] = None
        self.w2: Optional[torch.Tensor] = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {
            "w1.weight": ExpectedTensor((self.hidden, self.dim)),
            "w2.weight": ExpectedTensor((self.dim, self.hidden)),
            "w3.weight": ExpectedTensor((self.hidden, self.dim)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.w13 = torch.cat([as_compute(tensors["w1.weight"], self.env), as_compute(tensors["w3.weight"], self.env)])
        self.w2 = as_compute(tensors["w2.weight"], self.env)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        ops = self.env.ops
        # gate and up in one product over the stacked weight, the activation in its epilogue where the
        # kernel can (decode steps), else product [T, 2 * hidden] + SwiGLU kernel
        # the down projection is left to the norm that follows (see PendingProduct)
        return PendingProduct(ops.linear_swiglu(x, self.w13), self.w2)
