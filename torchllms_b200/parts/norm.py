"""Root-mean-square norm, fused with the residual sum that precedes it.

Reference: ``RMSNorm.forward`` (torchllms/models/networks.py:195-200) squares,
averages and rescales in float32, casts back to the activation dtype and then
multiplies by the weight.  Here the stream itself is float32, the pending
delta is added in float32, and the weight is applied before the single
rounding to the activation dtype; in float32 the two orders are the same
arithmetic.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..weights.loader import ExpectedTensor
from .base import BuildEnv, Norm, Residual, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, env: BuildEnv, *, dim: int, eps: float):
        self.env = env
        self.dim = int(dim)
        self.eps = float(eps)
        self.weight: Optional[torch.Tensor] = None

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {"weight": ExpectedTensor((self.dim,))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # Kept in 32-bit whatever the activation dtype: the kernel multiplies in 32-bit.
        self.weight = tensors["weight"].to(device=self.env.device, dtype=torch.float32).contiguous()

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = self.env.ops.rmsnorm(residual.h, residual.delta, self.weight, self.eps,
                                   out_dtype=self.env.dtype, rows=rows)
        if rows is None:
            residual.delta = None  # the kernel wrote h + delta back into the stream
        return out
