"""Strict loading of a model's tensors by name.

The reference loads with ``load_state_dict(strict=False, assign=True)``, only
warns about missing or unexpected keys and then fills whatever stayed
uninitialised with random numbers (torchllms/models/utils.py:107-128,
:141-164).  Here a checkpoint either provides exactly the tensors the model
declares, with the declared shapes, or loading stops with one error that
lists everything that is wrong.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from .safetensors_io import TensorSource


class WeightError(ValueError):
    """A checkpoint does not match the model: lists missing, unexpected and misshapen tensors."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 other: Optional[List[str]] = None):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other or [])
        lines = [f"{where}: the checkpoint does not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} expected {list(e)} found {list(f)}" for n, e, f in self.wrong_shape))
        for msg in self.other:
            lines.append("  " + msg)
        super().__init__("\n".join(lines))


@dataclass
class LazyTensor:
    """A tensor of known shape and stored dtype that is read only when asked for."""

    shape: Tuple[int, ...]
    dtype: torch.dtype
    fetch: Callable[[], torch.Tensor]

    def materialize(self) -> torch.Tensor:
        t = self.fetch()
        if tuple(t.shape) != tuple(self.shape):
            raise AssertionError(f"fetched shape {tuple(t.shape)} != declared {tuple(self.shape)}")
        return t

    @classmethod
    def of(cls, t: torch.Tensor) -> "LazyTensor":
        return cls(tuple(t.shape), t.dtype, lambda: t)

    def mapped(self, fn: Callable[[torch.Tensor], torch.Tensor],
               shape: Optional[Tuple[int, ...]] = None) -> "LazyTensor":
        inner = self.fetch
        return LazyTensor(tuple(shape or self.shape), self.dtype, lambda: fn(inner()))


@dataclass(frozen=True)
class ExpectedTensor:
    shape: Tuple[int, ...]
    # "float": any floating dtype is accepted and handed over as stored;
    # "int": an integer table, handed over as int32.
    family: str = "float"


def source_tensors(source: TensorSource) -> Dict[str, LazyTensor]:
    return {name: LazyTensor(source.shape(name), source.dtype(name),
                             (lambda n=name: source.get(n)))
            for name in source.names()}


def check_tensors(where: str, expected: Mapping[str, ExpectedTensor],
                  found: Mapping[str, LazyTensor], ignorable: Iterable[str] = ()) -> None:
    """Raise one :class:`WeightError` for every mismatch between the two sets."""
    ignorable = set(ignorable)
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected and n not in ignorable]
    wrong = [(n, tuple(e.shape), tuple(found[n].shape)) for n, e in expected.items()
             if n in found and tuple(found[n].shape) != tuple(e.shape)]
    other = []
    for n, e in expected.items():
        if n in found and n not in [w[0] for w in wrong]:
            is_float = found[n].dtype.is_floating_point
            if e.family == "float" and not is_float:
                other.append(f"{n}: expected a floating-point tensor, found {found[n].dtype}")
            if e.family == "int" and is_float:
                other.append(f"{n}: expected an integer table, found {found[n].dtype}")
    if missing or unexpected or wrong or other:
        raise WeightError(where, missing, unexpected, wrong, other)


def materialize(expected: Mapping[str, ExpectedTensor], found: Mapping[str, LazyTensor]) -> Dict[str, torch.Tensor]:
    """Fetch the expected tensors in their stored dtype (bfloat16 stays
    bfloat16, a tensor stored in 32-bit stays so); integer tables become int32.
    The parts decide later what their compute dtype needs."""
    out: Dict[str, torch.Tensor] = {}
    for name, e in expected.items():
        t = found[name].materialize()
        if e.family == "int":
            t = t.to(torch.int32)
        out[name] = t
    return out
