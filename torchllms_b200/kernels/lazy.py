"""Two small value types that let work be moved across the borders of parts without the parts
knowing of each other.

:class:`PendingProduct`
    A matrix product that has not been taken yet: ``x @ w.T``.  A mixer or a feed-forward may
    return its last projection this way.  Whoever consumes it decides how it is taken: the norm
    that follows can hand it to a kernel that adds the product to the residual stream and
    prepares the norm in its epilogue; anybody else calls :meth:`take`.

:class:`RowScaled`
    Rows whose RMS normalisation was deferred: ``x`` holds ``h * norm_weight`` (or anything
    computed from it by matrix products, which are linear in their input, e.g. float32 partial
    sums ``[splits, T, n]``), and the true value of row ``t`` is ``x[t] * scale[t]`` with
    ``scale[t] = rsqrt(sum_p ssq[t, p] / dim + eps)``.  The sum of squares may come in several
    parts (one per column slab of the kernel that produced ``h``); consumers add them up.  The
    kernels that end a chain of products (rotary encoding, the SwiGLU gate) apply the scale, in
    float32, where they convert to the activation dtype anyway.

The reference computes ``norm(x) @ W`` (torchllms/models/networks.py:195-200, :635-644); here
the same number is ``(x * w_norm) @ W * rsqrt(mean(x^2) + eps)``, which lets the kernel that
produces ``x`` finish without a pass over the whole row.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class PendingProduct:
    x: torch.Tensor          # [T, K], activation dtype
    w: torch.Tensor          # [N, K], the weight as nn.Linear keeps it

    def take(self, ops, partials_ok: bool = True):
        """The product as a tensor (or float32 partial sums when ``partials_ok``)."""
        return ops.linear(self.x, self.w, partials_ok=partials_ok)

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])


@dataclass
class RowScaled:
    x: torch.Tensor          # [T, n] in the activation dtype, or float32 partial sums [splits, T, n]
    ssq: torch.Tensor        # [T, parts] float32: parts of every row's sum of squares
    dim: int                 # how many elements each row's squares were summed over
    eps: float

    def follow(self, x: torch.Tensor) -> "RowScaled":
        """The same rows' scale on another tensor computed linearly from ``x``."""
        return RowScaled(x, self.ssq, self.dim, self.eps)

    def scale(self) -> torch.Tensor:
        """``[T]`` float32: what every row is still to be multiplied by (for plain PyTorch callers)."""
        return torch.rsqrt(self.ssq.float().sum(-1) / self.dim + self.eps)

    def resolve(self, dtype: torch.dtype) -> torch.Tensor:
        """The rows themselves, in ``dtype`` (plain PyTorch; no kernel of the package is involved)."""
        x = self.x.float().sum(0) if self.x.dim() == 3 else self.x.float()
        return (x * self.scale()[:, None]).to(dtype)
