"""Interfaces of the parts a layer is put together from, and their registries.

A layer is a *block* (the arrangement: where the norms sit, how the residual
is carried) over a *mixer* (what lets tokens see each other: attention here),
a *feed-forward* (dense here; experts elsewhere), *norms* and, inside the
mixer, a *position encoding*.  The reference hard-wires one such combination
(``TransformerBlock`` over ``Attention``, ``FeedForward``, ``RMSNorm`` and
``RotaryPositionalEmbeddings``, torchllms/models/networks.py:186-644) and hands
every part the whole parameter object.  Here each part is a class registered
under a kind name, built from plain numbers, and told nothing about the model
it sits in; the model spec picks kinds and numbers layer by layer.

What every part has in common (:class:`Part`):

``expected_tensors()``
    local tensor names -> :class:`~torchllms_b200.weights.loader.ExpectedTensor`.
``load(tensors)``
    receives exactly those tensors (CPU, as stored) and places them on the
    device in whatever packing its kernels want.

What each family adds is documented on its base class below.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Optional, Tuple

import torch

from ..weights.loader import ExpectedTensor
from .spec import PartSpec


@dataclass(frozen=True)
class BuildEnv:
    """What a part may know of its surroundings when it is built."""

    dim: int                 # width of the residual stream
    dtype: torch.dtype       # activation / weight dtype: torch.bfloat16 or torch.float32
    device: torch.device
    max_positions: int       # the longest sequence the engine will hold
    ops: Any                 # the kernel library (see torchllms_b200.kernels)


@dataclass(frozen=True)
class CacheNeed:
    """Paged key/value storage a mixer wants for every token of a request.

    ``kind`` is ``"full"`` (all keys stay) or ``"window"`` (only the last
    ``window`` keys are ever read, so older pages may be given back).  Runs
    with equal needs share one group of pages and one block table.
    """

    kind: str
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def __post_init__(self):
        if self.kind not in ("full", "window"):
            raise ValueError(f"cache kind must be 'full' or 'window', got {self.kind!r}")
        if (self.kind == "window") != (self.window is not None):
            raise ValueError("a window size goes with kind 'window' and only with it")


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (``shape`` elements of ``dtype``), kept in a slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    # True when forward() only enqueues work on the current stream with shapes that depend on the
    # step's token and request counts alone (no read-back, no host-side branching on device
    # data): such a part may be captured into a CUDA graph and replayed.
    graph_safe = False

    def expected_tensors(self) -> Dict[str, ExpectedTensor]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass

    def weight_bytes(self) -> int:
        """Bytes of the weights this part (and the parts inside it) reads in a step."""
        total = 0
        for v in vars(self).values():
            if isinstance(v, torch.Tensor) and v.is_floating_point():
                total += v.numel() * v.element_size()
            elif isinstance(v, Part):
                total += v.weight_bytes()
        return total


class Norm(Part):
    """``forward(residual, rows=None)``: folds the residual's pending delta into
    the stream (32-bit sum) and returns the normalised rows in the activation
    dtype; with ``rows`` (int32 indices) only those rows are produced and the
    stream is left as it was.

    The pending delta may be a tensor, float32 partial sums, or a
    :class:`~torchllms_b200.kernels.lazy.PendingProduct` (``ops.rmsnorm`` takes all three).  A
    norm with ``can_defer`` also accepts ``deferred_ok=True`` and may then return a
    :class:`~torchllms_b200.kernels.lazy.RowScaled` (rows weighted but not yet normalised, the
    scale to be applied by whoever consumes them); a block passes that flag only to such a norm
    and only when the part that reads the rows has ``takes_row_scaled``."""

    can_defer = False

    def forward(self, residual: "Residual", rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns a mixer's projected ``[T, (H + 2 KV) * hd]`` rows into position-aware
    queries and stores position-aware keys (and raw values) in the cache.

    ``encode_and_store(qkv, ctx, cache, n_heads, n_kv_heads, head_dim)`` returns
    ``q [T, H, hd]``; it writes K and V at ``cache.slot_mapping`` when
    ``cache.writes`` is true.  ``qkv`` may be float32 partial sums ``[splits, T, row]``, and, if the
    encoding sets ``takes_row_scaled``, a :class:`~torchllms_b200.kernels.lazy.RowScaled`."""

    takes_row_scaled = False

    def encode_and_store(self, qkv, ctx, cache, n_heads: int, n_kv_heads: int, head_dim: int):
        raise NotImplementedError


class Mixer(Part):
    """``forward(x [T, dim], ctx, cache) -> [T, dim]`` (activation dtype).

    ``x`` is a tensor unless the mixer sets ``takes_row_scaled`` (then it may be a
    :class:`~torchllms_b200.kernels.lazy.RowScaled`, which the kernel library's ``linear``,
    ``rope_kv_write`` and ``linear_swiglu`` accept in a tensor's place).  The result may be a
    :class:`~torchllms_b200.kernels.lazy.PendingProduct`: a last projection left for the norm that
    follows to take.

    ``cache_need()`` / ``state_need()`` tell the cache manager what one run of
    this mixer wants per request (either may be ``None``).  ``cache`` is the
    :class:`~torchllms_b200.cache.manager.RunCacheView` of the run being
    executed: page tensors, block table, slot mapping, and the state rows.
    A mixer with state must handle the portions of a request in order;
    ``ctx.fresh`` marks requests whose portion starts at position 0.
    """

    takes_row_scaled = False

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x [T, dim], ctx) -> [T, dim]`` (activation dtype); tokens do not interact.
    ``takes_row_scaled`` and a pending last projection as for a mixer."""

    takes_row_scaled = False

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of one layer.  ``forward(residual, ctx, cache)`` updates the
    residual (stream + pending delta) in place."""

    def forward(self, residual: "Residual", ctx, cache) -> None:
        raise NotImplementedError

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None


class Residual:
    """The residual stream ``h`` (float32, ``[T, dim]``) and a delta not yet added.

    Keeping the last delta pending lets the next norm kernel do ``h += delta``
    and the normalisation in one pass over the row.  The delta is ``[T, dim]`` in
    the activation dtype, or float32 partial sums ``[splits, T, dim]`` of a
    split-K product, which the norm kernel adds up as well, or a product not yet
    taken (:class:`~torchllms_b200.kernels.lazy.PendingProduct`), which the norm may
    hand to a kernel that adds it to ``h`` in its own epilogue.
    """

    __slots__ = ("h", "delta")

    def __init__(self, h: torch.Tensor, delta: Optional[torch.Tensor] = None):
        self.h = h
        self.delta = delta


# --------------------------------------------------------------------------- registries

class Registry:
    def __init__(self, family: str, base: type):
        self.family = family
        self.base = base
        self._kinds: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls: type) -> type:
            if not issubclass(cls, self.base):
                raise TypeError(f"{cls.__name__} must derive from {self.base.__name__} to be a {self.family}")
            self._kinds[kind] = cls
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def build(self, spec: PartSpec, env: BuildEnv):
        try:
            cls = self._kinds[spec.kind]
        except KeyError:
            known = ", ".join(sorted(self._kinds)) or "(none)"
            raise KeyError(f"unknown {self.family} kind {spec.kind!r}; registered: {known}") from None
        return cls(env, **spec.params)

    def kinds(self):
        return sorted(self._kinds)


NORMS = Registry("norm", Norm)
POSITION_ENCODINGS = Registry("position encoding", PositionEncoding)
MIXERS = Registry("mixer", Mixer)
FEED_FORWARDS = Registry("feed-forward", FeedForward)
BLOCKS = Registry("block", Block)

register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register


def as_compute(t: torch.Tensor, env: BuildEnv) -> torch.Tensor:
    """A matrix weight on the device in the activation dtype, contiguous."""
    return t.to(device=env.device, dtype=env.dtype).contiguous()
