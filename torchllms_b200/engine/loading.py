"""From a model folder (or a configuration and a seed) to a loaded :class:`Model`.

Reference: ``setup_model_and_tokenizer`` (torchllms/models/utils.py:18-93): read
the parameter file, apply keyword overrides, build the model, load the weights,
cast to the requested precision.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..config.registry import Architecture, get_architecture, load_config
from ..kernels import get_ops
from ..weights.loader import LazyTensor, WeightError, check_tensors, materialize, source_tensors
from ..weights.safetensors_io import TORCH_SUFFIXES, TensorSource
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; use 'bfloat16' or 'float32'") from None


def model_dir_of(path) -> Path:
    """A model folder, or a file inside one (the reference takes checkpoint file paths and
    reads the configuration beside the first, torchllms/models/utils.py:42-43)."""
    path = Path(path)
    return path if path.is_dir() else path.parent


def load_model(path, *, dtype="bfloat16", device="cuda", overrides: Optional[Mapping[str, Any]] = None,
               max_positions: Optional[int] = None, ops=None) -> Tuple[Architecture, Any, Model]:
    """``path`` is a model folder, a safetensors file, a ``torch.save``d checkpoint of plain tensors
    (the reference's ``consolidated.00.pth`` beside its ``params.json``), or a list of them: tensors of later
    entries replace those of earlier ones (the reference loads several checkpoint paths in order,
    torchllms/models/utils.py:102-130); the configuration is read beside the first."""
    paths = [path] if isinstance(path, (str, Path)) else list(path)
    folder = model_dir_of(paths[0])
    arch, config = load_config(folder, overrides)
    spec = arch.build_spec(config)
    model = Model(spec, dtype=parse_dtype(dtype), device=device, ops=ops or get_ops(),
                  max_positions=max_positions)
    found: Dict[str, LazyTensor] = {}
    for p in paths:
        p = Path(p)
        source = TensorSource(p if p.is_file() and p.suffix in (".safetensors",) + TORCH_SUFFIXES else model_dir_of(p))
        found.update(arch.adapt_tensors(config, source_tensors(source)))
    expected = model.expected_tensors()
    if (spec.tie_head and spec.head_tensor != spec.embedding_tensor
            and spec.head_tensor in found and spec.embedding_tensor in found):
        # A tied model stores one table.  A second copy is tolerated only if it is the same table.
        head, table = found[spec.head_tensor], found[spec.embedding_tensor]
        same = tuple(head.shape) == tuple(table.shape) and torch.equal(head.materialize(), table.materialize())
        if not same:
            raise WeightError(str(folder), [], [], [], [
                f"{spec.head_tensor}: the configuration ties the head to {spec.embedding_tensor}, "
                "but the checkpoint holds a different head"])
        del found[spec.head_tensor]
    check_tensors(str(folder), expected, found)
    model.load(materialize(expected, found))
    return arch, config, model


def random_model(config, seed: int, *, dtype="bfloat16", device="cuda", arch: Optional[Architecture] = None,
                 max_positions: Optional[int] = None, ops=None) -> Tuple[Architecture, Any, Model]:
    """Random weights drawn on ``device`` without a file (for models too large to write)."""
    arch = arch or get_architecture(config.architecture)
    model = Model(arch.build_spec(config), dtype=parse_dtype(dtype), device=device, ops=ops or get_ops(),
                  max_positions=max_positions)
    tensors: Dict[str, torch.Tensor] = dict(arch.random_tensors(config, seed, device=device, dtype=model.dtype))
    check_tensors("random weights", model.expected_tensors(), {k: LazyTensor.of(v) for k, v in tensors.items()})
    model.load(tensors)
    return arch, config, model
