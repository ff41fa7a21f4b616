"""Root-mean-square norm, fused with the residual sum that precedes it.

Reference: ``RMSNorm.forward`` (torchllms/models/networks.py:195-200) squares,
averages and rescales in float32, casts back to the activation dtype and then
multiplies by the weight.  Here the stream itself is float32, the pending
delta is added in float32, and the weight is applied before the single
rounding to the activation dtype; in float32 the two orders are the same
arithmetic.

In bfloat16, when the part that reads the rows feeds them to a matrix product
first (``deferred_ok``), the rows leave as ``bf16(h * weight)`` with their sums
of squares, and the scale ``rsqrt(mean(h^2) + eps)`` is applied to the product
(a product is linear in its input): the same number with one rounding moved.
That lets a pending product add itself to the stream and prepare these rows in
its own epilogue, so that no norm kernel stands between two products of a
decode step.  Prompt portions go through the norm kernel in the same deferred
form, so that one arithmetic holds however a request is cut.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels.lazy import PendingProduct
from ..weights.loader import ExpectedTensor
from .base import BuildEnv, Norm, Residual, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True
    can_defer = True

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

    def forward(self, residual: Residual, rows: Optional[torch.Tensor] = None, deferred_ok: bool = False):
        ops = self.env.ops
        # 32-bit mode keeps the reference's order of operations to the letter
        deferred = bool(deferred_ok and rows is None and self.env.dtype == torch.bfloat16)
        delta = residual.delta
        if deferred and isinstance(delta, PendingProduct) and ops.can_fuse_residual(delta, residual.h):
            out = ops.linear_residual_norm(delta, residual.h, self.weight, self.eps)   # h += product, in the product's kernel
            residual.delta = None
            return out
        if deferred:
            out = ops.rmsnorm(residual.h, delta, self.weight, self.eps, out_dtype=self.env.dtype, deferred=True)
        else:
            out = ops.rmsnorm(residual.h, delta, self.weight, self.eps, out_dtype=self.env.dtype, rows=rows)
        if rows is None:
            residual.delta = None  # the kernel wrote h + delta back into the stream
        return out
