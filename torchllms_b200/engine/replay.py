"""Trace replay: feed given token ids through the engine step by step and write logits.

It samples nothing and owns nothing: the model is built by the same loader, the
steps run through the same :class:`~torchllms_b200.engine.step.Engine` (cache,
step function, kernels) that generation uses.  The nearest thing in the
reference is the logit-capturing hook of its validation script
(torchllms/inference/validate_qwen3.py:203-237).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: each request's next tokens and the places among them whose logits
are wanted; all entries of a step run as one batch.  ``end``: requests that are
finished after this step; their pages and slot are given back.  For a step with
wanted places, ``<out>/<step>.f32`` holds the logits as little-endian float32
``[wanted, vocab]`` in the order of the entries and of ``want``.  After every
step ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path
from typing import Dict, Optional

import numpy as np
import torch

from .loading import load_model
from .step import Engine, StepEntry


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class Replayer:
    def __init__(self, model_dir, dtype: str, max_tokens: int, *, page_size: int = 16, device: str = "cuda",
                 max_num_seqs: int = 16, ops=None):
        from ..config.registry import load_config
        _arch, config = load_config(model_dir)
        # The pool is made for max_tokens, so the position table must reach as far as one
        # request could grow inside it, whatever the configuration's own limit says.
        max_positions = max(int(config.max_seq_len), round_up(max_tokens, page_size))
        _, self.config, model = load_model(model_dir, dtype=dtype, device=device, ops=ops,
                                           max_positions=max_positions)
        self.engine = Engine(model, page_size=page_size, pool_tokens=round_up(max_tokens, page_size),
                             max_num_seqs=max_num_seqs, max_len=max_positions,
                             max_step_tokens=max(round_up(max_tokens, page_size), 64))
        self.handles: Dict[str, int] = {}

    def run_step(self, record: dict) -> Optional[np.ndarray]:
        entries = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            tokens = [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            if rid not in self.handles:
                self.handles[rid] = self.engine.claim()
            entries.append(StepEntry(self.handles[rid], tokens, [int(w) for w in e.get("want", [])]))
        logits = self.engine.step(entries) if entries else None
        for rid in record.get("end", []):
            handle = self.handles.pop(str(rid), None)
            if handle is not None:
                self.engine.release(handle)
        if logits is None:
            return None
        host = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
        check = getattr(self.engine.model.ops, "check_status", None)
        if check is not None:
            check()          # the copy synchronised: a kernel that gave up a wait has said so by now
        return host


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    replayer = Replayer(args.model, args.dtype, args.max_tokens, page_size=args.page_size)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = replayer.run_step(record)
        if logits is not None:
            logits.tofile(out / f"{step}.f32")
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
