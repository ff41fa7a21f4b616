"""The model as data: which parts, with which numbers, in which order.

An architecture turns its configuration into a :class:`ModelSpec`.  The spec
names a kind for every part (looked up in the part registries) together with
the sizes and constants that part needs, layer by layer, so one model may mix
different mixers and feed-forwards.  The order in which layers run is a list
of :class:`RunEntry`: it may name a layer twice, and an entry may read the
cache that another entry writes.  Nothing here knows what a Llama is.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """A part's registered kind and its parameters (plain numbers and nested specs)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __getitem__(self, key: str) -> Any:
        try:
            return self.params[key]
        except KeyError:
            raise KeyError(f"part '{self.kind}' was given no parameter '{key}'") from None

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


def part(kind: str, **params: Any) -> PartSpec:
    return PartSpec(kind, params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer's own weights: ``name`` is the prefix of the layer's tensors (``layers.3``),
    ``block`` the arrangement.  The block's parameters carry everything inside it as nested
    specs (mixers, feed-forwards, norms, however many and wherever the block kind puts them),
    just as a mixer carries its position encoding; nothing outside the block kind knows what a
    layer is made of."""

    name: str
    block: PartSpec


@dataclass(frozen=True)
class RunEntry:
    """One run of a layer.  ``cache_of`` names the run (its index in the run
    order) whose cache this run reads instead of writing one of its own."""

    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    dim: int
    vocab_size: int
    max_positions: int
    embedding_tensor: str            # name of the [vocab, dim] table
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    final_norm_prefix: str           # prefix of the final norm's tensors
    head_tensor: str                 # name of the [vocab, dim] output matrix
    tie_head: bool = False           # the head is the embedding table; head_tensor is absent

    def __post_init__(self):
        n = len(self.layers)
        for i, run in enumerate(self.run_order):
            if not 0 <= run.layer < n:
                raise ValueError(f"run {i} names layer {run.layer}, but there are {n} layers")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(
                        f"run {i} reads the cache of run {run.cache_of}, which must come before it")
                if self.run_order[run.cache_of].cache_of is not None:
                    raise ValueError(
                        f"run {i} reads the cache of run {run.cache_of}, which owns none itself")
