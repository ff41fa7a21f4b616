"""Rotary position encoding with the llama3 frequency rescaling.

Reference: ``RotaryPositionalEmbeddings`` (torchllms/models/networks.py:204-352).
``rope_init`` (:252-282) builds ``theta_i = base^(-2i/hd)`` and, for
``rope_type == "llama3"``, rescales low frequencies by ``1/factor`` and blends
the middle band (:259-277); ``build_rope_cache`` (:284-297) tabulates
``cos(p * theta_i), sin(p * theta_i)`` in float32 for every position; ``forward``
(:321-352) rotates adjacent lanes ``(x[2i], x[2i+1])`` in float32.  Keys are
stored after rotation, values as they are (:551-553).

The table is built once on the host in float32, exactly as the reference does
it, and gathered by the kernel; the rotation itself runs in float32 in the
kernel that also writes K and V into their pages.
"""

from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch

from .base import BuildEnv, PositionEncoding, register_position_encoding


def rotary_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping[str, Any]] = None) -> torch.Tensor:
    """``[head_dim / 2]`` float32 angular frequencies (torchllms/models/networks.py:253-279)."""
    exponent = torch.arange(0, head_dim, 2)[: head_dim // 2].float() / head_dim
    freq = 1.0 / (theta ** exponent)
    scaling = dict(scaling or {})
    rope_type = scaling.get("rope_type", "default")
    if rope_type == "llama3":
        factor = scaling["factor"]
        low = scaling["low_freq_factor"]
        high = scaling["high_freq_factor"]
        original = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / freq
        scaled = torch.where(wavelen > original / low, freq / factor, freq)
        smooth = (original / wavelen - low) / (high - low)
        blended = (1 - smooth) * scaled / factor + smooth * scaled
        medium = ~(wavelen < original / high) & ~(wavelen > original / low)
        freq = torch.where(medium, blended, scaled)
    elif rope_type != "default":
        raise ValueError(f"unknown rope_type {rope_type!r}")
    return freq


def rotary_table(freq: torch.Tensor, max_positions: int) -> torch.Tensor:
    """``[max_positions, head_dim / 2, 2]`` float32 (cos, sin) (torchllms/models/networks.py:284-297)."""
    positions = torch.arange(max_positions, dtype=freq.dtype)
    angles = torch.einsum("i,j->ij", positions, freq).float()
    return torch.stack([torch.cos(angles), torch.sin(angles)], dim=-1).contiguous()


@register_position_encoding("rope")
class RotaryEncoding(PositionEncoding):
    """``pairing`` is ``"interleaved"`` (lanes 2i, 2i+1: the reference's and Meta's
    convention) or ``"half"`` (lanes i, i + hd/2: Hugging Face's)."""

    graph_safe = True
    takes_row_scaled = True      # the kernel scales every row before it rotates and stores it

    def __init__(self, env: BuildEnv, *, head_dim: int, theta: float,
                 scaling: Optional[Mapping[str, Any]] = None, pairing: str = "interleaved"):
        if pairing not in ("interleaved", "half"):
            raise ValueError(f"rope pairing must be 'interleaved' or 'half', got {pairing!r}")
        self.env = env
        self.head_dim = int(head_dim)
        self.pairing = pairing
        self.freq = rotary_frequencies(self.head_dim, float(theta), scaling)
        self.table = rotary_table(self.freq, env.max_positions).to(env.device)

    def weight_bytes(self) -> int:
        return 0  # the table is gathered by rows, not streamed

    def encode_and_store(self, qkv, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int):
        return self.env.ops.rope_kv_write(
            qkv, ctx.positions, self.table,
            n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
            interleaved=(self.pairing == "interleaved"),
            k_pages=cache.k_pages if cache.writes else None,
            v_pages=cache.v_pages if cache.writes else None,
            slot_mapping=cache.slot_mapping, page_size=cache.page_size, out_dtype=self.env.dtype)
