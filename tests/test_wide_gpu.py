"""The engine at the widths of the 8-billion-parameter shape (dim 4096, 32 heads of 128 over 8 kv
heads, feed-forward 14336, vocabulary 128256, llama3 rope scaling) against the plain
implementation, in 32-bit and in bfloat16.  Two layers instead of 32: every kernel runs at its
full width, and the plain implementation still finishes on the host in reasonable time.

First a few hand-cut steps through the engine in this process; then the four ways of cutting of
the replay tests (whole prompts, the last 32 tokens one by one, portions of changing size, up to
four live requests mixed in a pool that makes pages be used again) through ``bin/trace_run`` with
prompts of up to 700 tokens.  At this length the tcgen05 prefill attention runs several query
tiles per CTA at head_dim 128, the library product runs with more than 64 rows at K = 4096 and
14336, and the head product writes float32: paths that the tiny configurations reach only at
narrow widths.  The reference's own whole-prompt prefill is torchllms/inference/llm.py:1042-1068,
its one-by-one decoding :946-981; its logit gate is 1e-3 in 32-bit
(torchllms/inference/validate_qwen3.py:579-584), five times what is allowed here."""

import random

import numpy as np
import pytest
import torch

import traces
from helpers import make_tensors, run_trace, write_model_folder
from plain_llama import PlainModel, to_bfloat16_and_back

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 2,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": False, "max_position_embeddings": 1024,
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


# ---------------------------------------------------------------- the four cuttings at full width

WIDE_LENGTHS = {"a": 700, "b": 300, "c": 130, "d": 97, "e": 260}
THIN = 53                       # a row of logits is half a megabyte: wanted places are thinned out
WIDE_MODES = {
    "whole": dict(thin=THIN),
    "tail_one_by_one": dict(thin=THIN),
    "portions": dict(sizes=(2, 300, 5, 257, 96, 31, 130, 3, 128, 17), thin=THIN),
    "mixed": dict(chunks=(2, 5, 24, 96, 150, 260, 40), thin=THIN),
}
WIDE_F32_ATOL = 2e-4


def wide_requests():
    rng = random.Random(77)
    return {rid: [rng.randrange(WIDE["vocab_size"]) for _ in range(n)] for rid, n in WIDE_LENGTHS.items()}


@pytest.fixture(scope="module")
def wide_traces():
    reqs = wide_requests()
    built = {mode: getattr(traces, mode)(reqs, **kw) for mode, kw in WIDE_MODES.items()}
    wanted = {rid: set() for rid in reqs}
    for _steps, places, _peak in built.values():
        for rows in places.values():
            for rid, pos in rows:
                wanted[rid].add(pos)
    return reqs, built, {rid: sorted(v) for rid, v in wanted.items()}


@pytest.fixture(scope="module")
def wide_reference(wide, wide_traces):
    """Plain logits at every place any cutting wants, per dtype: {dtype: ({request: {position: row}}, tolerance)}."""
    reqs, _built, wanted = wide_traces
    out = {}
    for dtype in (torch.float32, torch.bfloat16):
        plain = PlainModel(wide[dtype])
        ref = {rid: plain.logits(reqs[rid], rows=wanted[rid]).numpy() for rid in reqs}
        tol = WIDE_F32_ATOL
        if dtype == torch.bfloat16:
            # as above: the engine may be off from float32 by one and a half times what the
            # emulation that rounds where the engine stores is off
            moved = max(float(np.abs(plain.logits(reqs[rid], stored=to_bfloat16_and_back, rows=wanted[rid]).numpy() - ref[rid]).max())
                        for rid in reqs)
            tol = 1.5 * moved
        out[dtype] = ({rid: {pos: ref[rid][i] for i, pos in enumerate(wanted[rid])} for rid in reqs}, tol)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", list(WIDE_MODES))
def test_wide_replay(wide, wide_traces, wide_reference, tmp_path, dtype, mode):
    _reqs, built, _wanted = wide_traces
    steps, places, peak = built[mode]
    ref, tol = wide_reference[dtype]
    if mode == "portions":
        assert max(len(e["tokens"]) for s in steps for e in s["entries"]) == 300
    if mode == "mixed":
        assert peak < sum(-(-n // 64) * 64 for n in WIDE_LENGTHS.values())       # pages have to be used again
        assert max(len(s["entries"]) for s in steps) == 4
    got = run_trace(wide[dtype], "float32" if dtype == torch.float32 else "bfloat16", steps, tmp_path / "out",
                    max_tokens=peak, timeout=1800)
    assert set(got) == set(places)
    worst, flips, rows_checked = 0.0, 0, 0
    for step, rows in places.items():
        want = np.stack([ref[rid][pos] for rid, pos in rows])
        assert got[step].shape == want.shape and np.isfinite(got[step]).all()
        err = np.abs(got[step] - want).max(axis=1)
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, (f"step {step}: first wrong row {bad[0]} = request/position {rows[bad[0]]}, "
                               f"error {err[bad[0]]:.3g} > {tol:.3g}")
        worst = max(worst, float(err.max()))
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2 * tol
        flips += int((np.argmax(got[step], 1)[clear] != np.argmax(want, 1)[clear]).sum())
        rows_checked += len(rows)
    assert flips == 0
    print(f"wide {dtype} {mode}: {len(steps)} steps, {rows_checked} rows, pool {peak} tokens, "
          f"worst error {worst:.3g} (allowed {tol:.3g})")
