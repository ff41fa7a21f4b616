"""The kernels at the widths of the 8-billion-parameter shape (dim 4096, 32 heads of 128 over 8 kv
heads, feed-forward 14336, vocabulary 128256, llama3 rope scaling) with two layers: portions,
decoded tokens and a mixed step against the plain implementation, in 32-bit and in bfloat16."""

import json

import numpy as np
import pytest
import torch

from helpers import make_tensors, write_model_folder
from plain_llama import PlainModel, to_bfloat16_and_back

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "max_position_embeddings": 512,
}


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    tensors = make_tensors(WIDE, 3, std=0.02, qk_std=0.04)
    out = {}
    for dtype in (torch.float32, torch.bfloat16):
        folder = write_model_folder(tmp_path_factory.mktemp(str(dtype).split(".")[-1]), WIDE, tensors, dtype)
        out[dtype] = folder
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_wide_model_in_portions_and_mixed_steps(wide, dtype):
    from torchllms_b200.engine.replay import Replayer
    folder = wide[dtype]
    g = torch.Generator().manual_seed(9)
    a = torch.randint(0, WIDE["vocab_size"], (75,), generator=g).tolist()
    b = torch.randint(0, WIDE["vocab_size"], (40,), generator=g).tolist()
    plain = PlainModel(folder)
    if dtype == torch.float32:
        ref = {"a": plain.logits(a).numpy(), "b": plain.logits(b).numpy()}
        tol = 2e-4          # logits of order 1; float32 sums over K = 14336 in another order
    else:
        # At this width thousands of sums per layer sit close enough to a bfloat16 rounding step that
        # another summation order flips them, so the engine and the emulation are two equally good
        # bfloat16 evaluations rather than near copies.  Both are therefore held against float32: the
        # engine may be off by at most one and a half times what the emulation (which rounds where
        # the engine stores) is off.  A dropped key or a wrong position moves these peaked logits
        # by several times that.
        ref = {"a": plain.logits(a).numpy(), "b": plain.logits(b).numpy()}
        emu = {"a": plain.logits(a, stored=to_bfloat16_and_back).numpy(), "b": plain.logits(b, stored=to_bfloat16_and_back).numpy()}
        moved = max(float(np.abs(emu[k] - ref[k]).max()) for k in ref)
        tol = 1.5 * moved
    rp = Replayer(folder, "float32" if dtype == torch.float32 else "bfloat16", 256)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [0, 24, 49]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[50:51], "want": [0]}, {"id": "b", "tokens": b[:33], "want": [32]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[51:53], "want": [0, 1]}, {"id": "b", "tokens": b[33:34], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "b", "tokens": b[34:], "want": [5]}, {"id": "a", "tokens": a[53:], "want": [21]}], "end": ["a", "b"]},
    ]
    places = {0: [("a", 0), ("a", 24), ("a", 49)], 1: [("a", 50), ("b", 32)], 2: [("a", 51), ("a", 52), ("b", 33)],
              3: [("b", 39), ("a", 74)]}
    worst = 0.0
    for s in steps:
        got = rp.run_step(s)
        want = np.stack([ref[r][p] for r, p in places[s["step"]]])
        err = np.abs(got - want).max(axis=1)
        assert (err <= tol).all(), (s["step"], places[s["step"]][int(np.argmax(err))], float(err.max()), tol)
        worst = max(worst, float(err.max()))
    # decoding on for a while, one token per step, two requests side by side (the graphed path in bfloat16)
    ha, hb = "c", "d"
    rp.run_step({"step": 10, "entries": [{"id": ha, "tokens": a[:20], "want": []}, {"id": hb, "tokens": b[:10], "want": []}], "end": []})
    for i in range(12):
        got = rp.run_step({"step": 11 + i, "entries": [{"id": ha, "tokens": [a[20 + i]], "want": [0]},
                                                       {"id": hb, "tokens": [b[10 + i]], "want": [0]}], "end": []})
        want = np.stack([ref["a"][20 + i], ref["b"][10 + i]])
        err = np.abs(got - want).max()
        assert err <= tol, (i, float(err), tol)
    print(f"wide {dtype}: worst error {worst:.3g}, allowed {tol:.3g}")
