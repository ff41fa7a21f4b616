"""Pre-norm residual block.

Reference: ``TransformerBlock.forward`` (torchllms/models/networks.py:635-644):
``h = x + mixer(norm1(x)); out = h + ffn(norm2(h))``.  The sums are left pending
on the residual so the following norm adds them in 32-bit in the same pass.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..weights.loader import ExpectedTensor
from .base import FEED_FORWARDS, MIXERS, NORMS, Block, BuildEnv, Residual, register_block
from .spec import PartSpec


@register_block("prenorm")
class PreNormBlock(Block):
    """Sub-part tensor prefixes are parameters, so the block does not know whose names they are."""

    def __init__(self, env: BuildEnv, *, mixer: PartSpec, feed_forward: PartSpec,
                 mixer_norm: PartSpec, ffn_norm: PartSpec,
                 mixer_prefix: str, ffn_prefix: str, mixer_norm_prefix: str, ffn_norm_prefix: str):
        self.env = env
        self.mixer = MIXERS.build(mixer, env)
        self.feed_forward = FEED_FORWARDS.build(feed_forward, env)
        self.mixer_norm = NORMS.build(mixer_norm, env)
        self.ffn_norm = NORMS.build(ffn_norm, env)
        self.graph_safe = all(x.graph_safe for x in (self.mixer, self.feed_forward, self.mixer_norm, self.ffn_norm))
        self._subparts = ((mixer_prefix, self.mixer), (ffn_prefix, self.feed_forward),
                          (mixer_norm_prefix, self.mixer_norm), (ffn_norm_prefix, self.ffn_norm))

    def cache_need(self):
        return self.mixer.cache_need()

    def state_need(self):
        return self.mixer.state_need()

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for prefix, sub in self._subparts:
            for name, e in sub.expected_tensors().items():
                out[f"{prefix}.{name}"] = e
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for prefix, sub in self._subparts:
            sub.load({name: tensors[f"{prefix}.{name}"] for name in sub.expected_tensors()})

    def forward(self, residual: Residual, ctx, cache) -> None:
        x = self._normed(self.mixer_norm, self.mixer, residual)
        residual.delta = self.mixer.forward(x, ctx, cache)
        x = self._normed(self.ffn_norm, self.feed_forward, residual)
        residual.delta = self.feed_forward.forward(x, ctx)

    @staticmethod
    def _normed(norm, reader, residual: Residual):
        """The rows for ``reader``: with their normalisation deferred where both sides can."""
        if norm.can_defer and reader.takes_row_scaled:
            return norm.forward(residual, deferred_ok=True)
        return norm.forward(residual)
