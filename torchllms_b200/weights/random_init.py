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


def main(argv=None) -> None:
    """``python -m torchllms_b200.weights.random_init --config config.json --seed 0 --out DIR``"""
    import argparse

    from ..config.registry import architecture_of, load_config
    from ..engine.loading import parse_dtype

    p = argparse.ArgumentParser(description="Write a model folder with random weights for a configuration.")
    p.add_argument("--config", required=True, help="A config.json or params.json, or a folder that holds one.")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--out", required=True, help="Folder to write config.json and model.safetensors into.")
    p.add_argument("--dtype", default="bfloat16", help="Stored dtype: bfloat16 or float32.")
    args = p.parse_args(argv)
    src = Path(args.config)
    if src.is_dir():
        arch, config = load_config(src)
    else:
        with open(src) as f:
            raw = json.load(f)
        kind = "params.json" if "dim" in raw and "hidden_size" not in raw else "config.json"
        arch = architecture_of(raw, kind)
        config = arch.parse_config(raw, str(src))
    folder = write_random_model(args.out, config, args.seed, dtype=parse_dtype(args.dtype), arch=arch)
    print(folder)


if __name__ == "__main__":
    main()
