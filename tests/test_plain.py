"""The plain implementation against the outputs of the reference's own model code (recorded once
by tests/golden/make_golden.py), and against the engine's independent host-side formulas."""

import json
import math
from pathlib import Path

import pytest
import torch

import plain_llama
from helpers import TINY, hugging_face_names, make_tensors, write_model_folder

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_reproduces_the_reference_model(tmp_path, name):
    rec = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    cfg, seed, _ = TINY[name]
    assert rec["config"] == cfg and rec["seed"] == seed
    assert rec["max_diff_to_plain"] < 1e-5          # what the recording run itself saw
    plain = plain_llama.PlainModel(write_model_folder(tmp_path, cfg, make_tensors(cfg, seed, std=rec["std"], qk_std=rec["qk_std"])))
    for p in rec["prompts"]:
        logits = plain.logits(p["tokens"])
        rows = logits[[0, len(p["tokens"]) // 2, -1]][:, :len(p["logits_head"][0])]
        assert (rows - torch.tensor(p["logits_head"])).abs().max() < 1e-5
        assert (logits.double().sum(-1) - torch.tensor(p["logit_sum"], dtype=torch.float64)).abs().max() < 1e-3
        assert logits.argmax(-1).tolist() == p["argmax"]


@pytest.mark.parametrize("name", ["A", "B"])
def test_hugging_face_row_order_is_the_reference_converters(tmp_path, name):
    """The same tensors under Hugging Face names mean another model (their q and k rows are then
    in half-split order).  The record's ``hf`` entry is what the reference computes after its own
    converter has permuted them (torchllms/models/checkpoint_converter.py:96-108, :172-178); the
    plain implementation, with a permutation written on its own, and the engine, with its
    ``adapt_tensors``, must both land there."""
    from torch_ops import TorchOps
    from torchllms_b200.engine.replay import Replayer
    rec = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    cfg, seed, page = TINY[name]
    assert rec["hf"]["max_diff_to_plain"] < 1e-5
    folder = write_model_folder(tmp_path, cfg, hugging_face_names(make_tensors(cfg, seed, std=rec["std"], qk_std=rec["qk_std"])))
    plain = plain_llama.PlainModel(folder)
    engine = Replayer(folder, "float32", 256, page_size=page, device="cpu", ops=TorchOps())
    for i, (p, native) in enumerate(zip(rec["hf"]["prompts"], rec["prompts"])):
        toks = p["tokens"]
        got = engine.run_step({"step": i, "entries": [{"id": str(i), "tokens": toks, "want": list(range(len(toks)))}], "end": [str(i)]})
        for logits in (plain.logits(toks), torch.from_numpy(got)):
            rows = logits[[0, len(toks) // 2, -1]][:, :len(p["logits_head"][0])]
            assert (rows - torch.tensor(p["logits_head"])).abs().max() < 2e-5
            assert (logits.double().sum(-1) - torch.tensor(p["logit_sum"], dtype=torch.float64)).abs().max() < 2e-3
            assert logits.argmax(-1).tolist() == p["argmax"]
        if len(toks) > 1:
            assert p["logit_sum"][-1] != native["logit_sum"][-1]      # not the model the native names give


def test_rope_frequencies_agree_with_the_engines_table():
    from torchllms_b200.parts.rope import rotary_frequencies, rotary_table
    for hd, theta, scaling in ((16, 10000.0, None), (32, 500000.0, TINY["B"][0]["rope_scaling"]),
                               (128, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})):
        a = plain_llama.rope_frequencies(hd, theta, scaling)
        b = rotary_frequencies(hd, theta, scaling)
        assert torch.equal(a, b)
        cos, sin = plain_llama.rope_angles(a, torch.arange(300))
        table = rotary_table(b, 300)
        assert torch.equal(table[..., 0], cos) and torch.equal(table[..., 1], sin)
    scaled = plain_llama.rope_frequencies(128, 500000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
    plain = plain_llama.rope_frequencies(128, 500000.0, None)
    assert torch.equal(scaled[:20], plain[:20])                      # short waves untouched
    assert torch.allclose(scaled[-1], plain[-1] / 8)                 # long waves divided by the factor
    mid = (scaled != plain) & ~torch.isclose(scaled, plain / 8)
    assert mid.any()                                                 # and a blended band between


def test_rope_rotates_adjacent_lanes():
    x = torch.tensor([[[1.0, 0.0, 0.0, 2.0]]])                       # one token, one head, two pairs
    cos = torch.tensor([[0.0, 1.0]])
    sin = torch.tensor([[1.0, 0.0]])
    out = plain_llama.apply_rope(x, cos, sin)
    assert out.flatten().tolist() == [0.0, 1.0, 0.0, 2.0]            # first pair turned a quarter, second left alone


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    S, H, KV, hd = 6, 4, 2, 8
    q, k, v = torch.randn(S, H, hd), torch.randn(S, KV, hd), torch.randn(S, KV, hd)
    out = plain_llama.causal_attention(q, k, v).view(S, H, hd)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])    # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, -9.0
    out2 = plain_llama.causal_attention(q, k2, v2).view(S, H, hd)
    assert torch.equal(out[:4], out2[:4])                            # later keys never reach earlier queries
    w = plain_llama.causal_attention(q, k, v, window=1).view(S, H, hd)
    assert torch.allclose(w[:, 0], v[:, 0]) and torch.allclose(w[:, 2], v[:, 1])          # window 1: itself only
    s = (q[5, 1] @ k[:, 0].T) / math.sqrt(hd)
    assert torch.allclose(out[5, 1], torch.softmax(s, 0) @ v[:, 0], atol=1e-6)


def test_norm_and_ffn_formulas():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    got = plain_llama.rms_norm(x, w, 0.0)
    assert torch.allclose(got, torch.tensor([[3 / math.sqrt(12.5) * 2, 4 / math.sqrt(12.5) * 0.5]]))
    w1, w2, w3 = torch.tensor([[1.0, 0.0]]), torch.tensor([[2.0], [0.0]]), torch.tensor([[0.0, 1.0]])
    y = plain_llama.swiglu_ffn(x, w1, w2, w3)
    silu3 = 3 / (1 + math.exp(-3))
    assert torch.allclose(y, torch.tensor([[2 * silu3 * 4, 0.0]]))
