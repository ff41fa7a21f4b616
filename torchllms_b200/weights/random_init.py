"""Random-weights mode: write a model folder from a configuration and a seed.

The reference initialises whatever a checkpoint did not provide
(torchllms/models/utils.py:141-164, :197-214).  Here random weights are an
explicit mode that produces an ordinary model folder (``config.json`` and
``model.safetensors``), which then loads like any other.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Optional

import torch

from ..config.registry import Architecture, get_architecture
from .safetensors_io import write_safetensors


def write_random_model(out_dir, config, seed: int, *, dtype: torch.dtype = torch.float32,
                       arch: Optional[Architecture] = None, **init) -> Path:
    """Draw the architecture's tensors with one seeded generator and store them.

    ``dtype`` is the stored dtype of every tensor.  Returns the folder."""
    arch = arch or get_architecture(config.architecture)
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    with open(out_dir / "config.json", "w") as f:
        json.dump(config.to_hf(), f, indent=1)
    write_safetensors(out_dir / "model.safetensors",
                      arch.random_tensors(config, seed, device="cpu", dtype=dtype, **init),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
