"""Trace replay through bin/trace_run against the plain implementation: every way of cutting
and batching gives the same logits, in 32-bit and in bfloat16."""

import random

import numpy as np
import pytest
import torch

import traces
from helpers import TINY, tiny_folder
from helpers import run_trace
from plain_llama import PlainModel, to_bfloat16_and_back

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [1, 7, 33, 64, 97, 120, 50], "B": [2, 5, 17, 40, 100, 200, 65, 129],
           "C": [300, 97, 513, 130, 700, 64, 260], "D": [3, 50, 131, 64, 17, 90, 2, 158]}
# configuration C is there for long portions (the tcgen05 prefill kernel takes 96 tokens and more,
# 256 to a CTA): its cuttings include them
MODE_ARGS = {("C", "portions"): dict(sizes=(2, 130, 5, 257, 96, 31, 300, 3, 128, 17)),
             ("C", "mixed"): dict(chunks=(2, 5, 24, 96, 150, 260, 40))}
# float32: the reference's own gate is 1e-3 (torchllms/inference/validate_qwen3.py:579-584); these
# models are tiny, so a tenth of it.
# bfloat16: weights are stored in bfloat16 and read exactly by both sides, and the plain
# implementation rounds every intermediate where the engine stores one.  What is left: a sum taken
# in another order (other tiles, keys split over warps or CTAs) lands on the other side of a
# bfloat16 rounding step now and then, and one such flip then travels through these deliberately
# peaked models like any bfloat16 error does (each kernel alone was measured against float64:
# its error is exactly that of rounding the true result once).  So the yard-stick is how much
# bfloat16 storage itself moves these logits (plain-with-rounding against plain float32, computed
# per model below): the engine must stay within half of that from the emulation.  Measured on a
# B200: 0.1 to 0.26 of it, depending on the cutting; a dropped key, a stale page or a wrong
# position moves logits by several times the yard-stick (the float32 runs would catch them first).
F32_ATOL = 1e-4
BF16_SHARE = 0.5


def requests_for(name):
    cfg, seed, _ = TINY[name]
    rng = random.Random(seed + 100)
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in TINY:
        for dtype in ("float32", "bfloat16"):
            store = torch.float32 if dtype == "float32" else torch.bfloat16
            folder = tiny_folder(tmp_path_factory.mktemp(f"{name}_{dtype}"), name, dtype=store)
            reqs = requests_for(name)
            plain = PlainModel(folder)
            # bfloat16 is compared with the plain implementation rounding where the engine stores
            if dtype == "float32":
                ref = {rid: plain.logits(toks).numpy() for rid, toks in reqs.items()}
                tol = F32_ATOL
            else:
                ref = {rid: plain.logits(toks, stored=to_bfloat16_and_back).numpy() for rid, toks in reqs.items()}
                moved = max(float(np.abs(ref[rid] - plain.logits(toks).numpy()).max()) for rid, toks in reqs.items())
                tol = BF16_SHARE * moved
            out[(name, dtype)] = (folder, reqs, ref, tol)
    return out


def compare(got, places, ref, tol):
    assert set(got) == set(places)
    worst = 0.0
    flips = 0
    for step, rows in places.items():
        want = np.stack([ref[rid][pos] for rid, pos in rows])
        assert got[step].shape == want.shape
        assert np.isfinite(got[step]).all()
        err = np.abs(got[step] - want).max(axis=1)
        bad = np.nonzero(err > tol)[0]
        assert bad.size == 0, (f"step {step}: first wrong row {bad[0]} = request/position {rows[bad[0]]}, "
                               f"error {err[bad[0]]:.3g} > {tol:.3g}")
        worst = max(worst, float(err.max()))
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2 * tol
        flips += int((np.argmax(got[step], 1)[clear] != np.argmax(want, 1)[clear]).sum())
    assert flips == 0
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail_one_by_one", "portions", "mixed"])
def test_replay(setups, tmp_path, name, dtype, mode):
    folder, reqs, ref, tol = setups[(name, dtype)]
    steps, places, peak = getattr(traces, mode)(reqs, **MODE_ARGS.get((name, mode), {}))
    got = run_trace(folder, dtype, steps, tmp_path / "out", max_tokens=peak)
    worst = compare(got, places, ref, tol)
    print(f"{name} {dtype} {mode}: {len(steps)} steps, pool {peak} tokens, worst error {worst:.3g} (allowed {tol:.3g})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_first_tokens_and_long_decoding(setups, tmp_path, dtype):
    """The first tokens of a sequence one by one from an empty cache, then decoding on for long."""
    folder, reqs, ref, tol = setups[("B", dtype)]
    rid = "r5"                                   # 200 tokens
    toks = reqs[rid]
    steps = [{"step": i, "entries": [{"id": rid, "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    steps[-1]["end"] = [rid]
    places = {i: [(rid, i)] for i in range(len(toks))}
    got = run_trace(folder, dtype, steps, tmp_path / "out", max_tokens=256)
    compare(got, places, ref, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_decoding_past_a_context_bound(tmp_path, dtype):
    """Decode steps plan their attention (over how many CTAs the keys are split) for the power of two
    that holds the longest context, and are recorded once per such bound.  A request that grows from
    990 to 1,070 tokens one by one crosses the bound at 1,024 beside a short request: other plan,
    other recorded step, same logits."""
    from helpers import TINY_C, make_tensors, write_model_folder
    cfg = dict(TINY_C, max_position_embeddings=4096)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = write_model_folder(tmp_path / "tiny_long", cfg, make_tensors(cfg, 5, std=0.05, qk_std=0.25), store)
    rng = random.Random(11)
    reqs = {"long": [rng.randrange(cfg["vocab_size"]) for _ in range(1070)],
            "short": [rng.randrange(cfg["vocab_size"]) for _ in range(120)]}
    plain = PlainModel(folder)
    if dtype == "float32":
        ref = {rid: plain.logits(t).numpy() for rid, t in reqs.items()}
        tol = F32_ATOL
    else:
        ref = {rid: plain.logits(t, stored=to_bfloat16_and_back).numpy() for rid, t in reqs.items()}
        tol = BF16_SHARE * max(float(np.abs(ref[rid] - plain.logits(t).numpy()).max()) for rid, t in reqs.items())
    head = {"long": 990, "short": 40}
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": reqs["long"][:990], "want": [989]}], "end": []},
             {"step": 1, "entries": [{"id": "short", "tokens": reqs["short"][:40], "want": [39]}], "end": []}]
    places = {0: [("long", 989)], 1: [("short", 39)]}
    for i in range(80):
        step = len(steps)
        steps.append({"step": step, "entries": [{"id": "long", "tokens": [reqs["long"][990 + i]], "want": [0]},
                                                {"id": "short", "tokens": [reqs["short"][40 + i]], "want": [0]}],
                      "end": ["long", "short"] if i == 79 else []})
        places[step] = [("long", 990 + i), ("short", 40 + i)]
    got = run_trace(folder, dtype, steps, tmp_path / "out", max_tokens=1088 + 128)
    compare(got, places, ref, tol)
