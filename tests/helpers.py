"""Shared fixtures of the tests: tiny configurations that differ in every size and option (two for
everything, a third for the kernels that want heads of 64, a fourth of awkward sizes),
model folders with random weights, and traces for the replay program."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent

# Hugging Face style config.json contents.  A: grouped heads (2 per kv head), untied head, plain
# rope.  B: one kv head for three query heads, widths that are no power of two, tied head,
# llama3-scaled rope, another eps, a vocabulary that is no multiple of anything.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 192,
    "vocab_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "tie_word_embeddings": False, "max_position_embeddings": 128,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256,
    "vocab_size": 1000, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": True, "max_position_embeddings": 256,
}
# A third one for what the two above cannot reach: heads of 64 (the TMA-fed decode kernel and the
# tcgen05 prefill kernel take 64 and 128 only), a feed-forward width that the gated product takes,
# and room for prompts of several hundred tokens.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320,
    "vocab_size": 777, "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "rope_scaling": None,
    "tie_word_embeddings": False, "max_position_embeddings": 1024,
}
# A fourth one of awkward sizes: a width that is no multiple of four (the kernels' scalar forms, and
# products whose inner size the tensor-core kernel refuses), heads of 48 in groups of three, a
# feed-forward width and a vocabulary that are multiples of nothing, other constants everywhere.
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 102, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 166,
    "vocab_size": 1003, "rms_norm_eps": 1e-4, "rope_theta": 1234.5,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 2.0, "high_freq_factor": 8.0,
                     "original_max_position_embeddings": 32},
    "tie_word_embeddings": False, "max_position_embeddings": 160,
}
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16), "D": (TINY_D, 3, 4)}   # name -> (config, seed, page size)


def tensor_table(cfg: dict) -> List[tuple]:
    d, hd = cfg["hidden_size"], cfg["head_dim"]
    q, kv, f, v = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd, cfg["intermediate_size"], cfg["vocab_size"]
    rows = [("tok_embeddings.weight", (v, d), "m")]
    for i in range(cfg["num_hidden_layers"]):
        p = f"layers.{i}"
        rows += [(f"{p}.attention.wq.weight", (q, d), "qk"), (f"{p}.attention.wk.weight", (kv, d), "qk"),
                 (f"{p}.attention.wv.weight", (kv, d), "m"), (f"{p}.attention.wo.weight", (d, q), "m"),
                 (f"{p}.feed_forward.w1.weight", (f, d), "m"), (f"{p}.feed_forward.w2.weight", (d, f), "m"),
                 (f"{p}.feed_forward.w3.weight", (f, d), "m"),
                 (f"{p}.attention_norm.weight", (d,), "n"), (f"{p}.ffn_norm.weight", (d,), "n")]
    rows.append(("norm.weight", (d,), "n"))
    if not cfg["tie_word_embeddings"]:
        rows.append(("output.weight", (v, d), "m"))
    return rows


def make_tensors(cfg: dict, seed: int, *, std: float = 0.02, qk_std: Optional[float] = None) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under torchllms names.  ``qk_std`` makes the query and key
    projections larger so that attention is peaked and a single wrong key changes the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape, kind in tensor_table(cfg):
        t = torch.randn(shape, generator=g)
        if kind == "n":
            out[name] = 1.0 + 0.1 * t
        else:
            out[name] = t * (qk_std if (kind == "qk" and qk_std) else std)
    return out


_TO_HF_LAYER = {"attention.wq.weight": "self_attn.q_proj.weight", "attention.wk.weight": "self_attn.k_proj.weight",
                "attention.wv.weight": "self_attn.v_proj.weight", "attention.wo.weight": "self_attn.o_proj.weight",
                "feed_forward.w1.weight": "mlp.gate_proj.weight", "feed_forward.w3.weight": "mlp.up_proj.weight",
                "feed_forward.w2.weight": "mlp.down_proj.weight", "attention_norm.weight": "input_layernorm.weight",
                "ffn_norm.weight": "post_attention_layernorm.weight"}
_TO_HF_TOP = {"tok_embeddings.weight": "model.embed_tokens.weight", "norm.weight": "model.norm.weight",
              "output.weight": "lm_head.weight"}


def hugging_face_names(tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """The same tensors under Hugging Face names, values untouched (so the rows of q and k now
    stand in Hugging Face's order: a head's first halves, then its second halves)."""
    out = {}
    for name, t in tensors.items():
        if name.startswith("layers."):
            _, i, rest = name.split(".", 2)
            out[f"model.layers.{i}.{_TO_HF_LAYER[rest]}"] = t
        else:
            out[_TO_HF_TOP[name]] = t
    return out


def write_model_folder(folder, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> Path:
    """Tests write their folders with the ``safetensors`` package, not with the engine's writer."""
    from safetensors.torch import save_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: (v.to(dtype) if v.is_floating_point() else v).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def tiny_folder(tmp, name: str, *, sharp: bool = True, dtype=torch.float32) -> Path:
    cfg, seed, _ = TINY[name]
    return write_model_folder(Path(tmp) / f"tiny_{name}", cfg,
                              make_tensors(cfg, seed, std=0.05 if sharp else 0.02, qk_std=0.25 if sharp else None), dtype)


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def run_trace(model_dir, dtype: str, steps: Sequence[dict], out_dir, max_tokens: int, *, timeout=900,
              user: Optional[int] = None, cwd=None, vocab: Optional[int] = None) -> Dict[int, np.ndarray]:
    """Run bin/trace_run as a child process; returns {step: logits [wanted, vocab]}."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    cmd = [str((Path(cwd) if cwd else ROOT) / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    text = "".join(json.dumps(s) + "\n" for s in steps)
    env = dict(os.environ)
    env["TORCHLLMS_B200_PYTHON"] = sys.executable
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited {proc.returncode}\nstdout:\n{proc.stdout[-2000:]}\nstderr:\n{proc.stderr[-4000:]}")
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "one 'done' line per step, in order"
    if vocab is None:
        vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    result = {}
    for s in steps:
        n_want = sum(len(e.get("want", [])) for e in s["entries"])
        path = out_dir / f"{s['step']}.f32"
        if n_want:
            result[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n_want, vocab)
        else:
            assert not path.exists()
    return result
