"""Schedules and sizes on the GPU that the replay traces do not reach: an engine whose limit is
shorter than the model's position table, more live requests than one tile of the small-batch
product holds, and launching ahead while pages run out.

The reference requires every live request in every forward and refuses more than ``max_bsz`` of
them (torchllms/models/networks.py:984-990, torchllms/inference/llm.py:883-886); this engine
takes any subset and any number up to its slots, so both ends are tested here."""

import random

import numpy as np
import pytest
import torch

from helpers import TINY, tiny_folder
from plain_llama import PlainModel, to_bfloat16_and_back

pytestmark = pytest.mark.gpu


def reference(folder, reqs, dtype):
    """Plain logits per request and the tolerance of the replay tests for this dtype."""
    plain = PlainModel(folder)
    if dtype == "float32":
        return {rid: plain.logits(t).numpy() for rid, t in reqs.items()}, 1e-4
    ref = {rid: plain.logits(t, stored=to_bfloat16_and_back).numpy() for rid, t in reqs.items()}
    moved = max(float(np.abs(ref[rid] - plain.logits(t).numpy()).max()) for rid, t in reqs.items())
    return ref, 0.5 * moved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_engine_shorter_than_the_position_table_runs_mixed_steps(tmp_path, dtype):
    """Block tables are as wide as the engine's limit (here 384 of the model's 1,024 positions):
    the decode rows of a mixed step must plan for the engine's bound."""
    from torchllms_b200.engine.loading import load_model
    from torchllms_b200.engine.step import Engine, StepEntry
    cfg, _seed, page = TINY["C"]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = tiny_folder(tmp_path, "C", dtype=store)
    rng = random.Random(4)
    reqs = {"a": [rng.randrange(cfg["vocab_size"]) for _ in range(200)], "b": [rng.randrange(cfg["vocab_size"]) for _ in range(150)]}
    ref, tol = reference(folder, reqs, dtype)
    _, _, model = load_model(folder, dtype=dtype, device="cuda")
    assert model.max_positions == 1024
    eng = Engine(model, page_size=page, pool_tokens=768, max_num_seqs=4, max_len=384, max_step_tokens=256)
    a, b = eng.claim(), eng.claim()
    eng.step([StepEntry(a, reqs["a"][:180], [])])
    for i in range(3):
        # one decoded token of a beside a portion of b (long enough for the prefill kernel the first time), b first
        n = (120, 2, 20)[i]
        start = (0, 120, 122)[i]
        got = eng.step([StepEntry(b, reqs["b"][start:start + n], [n - 1]), StepEntry(a, [reqs["a"][180 + i]], [0])])
        want = np.stack([ref["b"][start + n - 1], ref["a"][180 + i]])
        err = float(np.abs(got.cpu().numpy() - want).max())
        assert err <= tol, (i, err, tol)
    model.ops.check_status()
    eng.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eighty_live_requests_decode_side_by_side(tmp_path, dtype):
    """More rows than the small-batch tensor-core product takes (64): decode steps of 80 requests
    leave it for the library product, and their recorded graphs are keyed like any other."""
    from torchllms_b200.engine.replay import Replayer
    cfg, _seed, page = TINY["C"]
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = tiny_folder(tmp_path, "C", dtype=store)
    rng = random.Random(8)
    n_req, n_decode = 80, 6
    reqs = {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(rng.randrange(3, 70) + n_decode)] for i in range(n_req)}
    ref, tol = reference(folder, reqs, dtype)
    total = sum(-(-len(t) // 64) * 64 for t in reqs.values())
    rp = Replayer(folder, dtype, total, page_size=page, max_num_seqs=96)
    ids = list(reqs)
    for lo in range(0, n_req, 20):                      # prompts, twenty requests to a step
        rp.run_step({"step": lo, "entries": [{"id": r, "tokens": reqs[r][:-n_decode], "want": []} for r in ids[lo:lo + 20]], "end": []})
    worst = 0.0
    for k in range(n_decode):
        live = ids if k < 4 else ids[:70]               # ten leave: another shape, another recorded step
        rec = {"step": 100 + k, "entries": [{"id": r, "tokens": [reqs[r][len(reqs[r]) - n_decode + k]], "want": [0]} for r in live],
               "end": ids[70:] if k == 3 else []}
        got = rp.run_step(rec)
        want = np.stack([ref[r][len(reqs[r]) - n_decode + k] for r in live])
        err = np.abs(got - want).max(axis=1)
        assert (err <= tol).all(), (k, live[int(np.argmax(err))], float(err.max()), tol)
        worst = max(worst, float(err.max()))
    rp.engine.cache.check_invariants()
    if dtype == "bfloat16":
        assert rp.engine.graph_replays > 0
    print(f"80 requests {dtype}: worst error {worst:.3g} (allowed {tol:.3g})")


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_launching_ahead_while_pages_run_out(tmp_path, precision):
    """A pool so tight that running requests are pre-empted and recomputed: steps launched ahead
    of their tokens (and called off when pages run out) give the tokens of the step-by-step way."""
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY["B"]
    folder = tiny_folder(tmp_path, "B")
    rng = random.Random(21)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (30, 9, 44, 17, 25, 5)]
    per_token = cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * (4 if precision == "float32" else 2)
    pool_tokens = 18 * page                              # 144 tokens: the longest request (44 + 48) fits; four at once do not
    kw = dict(precision=precision, max_len=256, max_bsz=4, page_size=page, max_num_batched_tokens=64, prefill_chunk=24,
              kv_memory_gb=pool_tokens * per_token / 2 ** 30)
    for sampling in (dict(), dict(temperature=0.8, seed=3)):
        ahead, stepwise = LLM(folder, look_ahead=True, **kw), LLM(folder, look_ahead=False, **kw)
        assert abs(ahead.engine.cache.groups[0].allocator.n_pages - pool_tokens // page) <= 1
        got = ahead.generate(prompt_token_ids=prompts, max_new_tokens=48, **sampling)
        want = stepwise.generate(prompt_token_ids=prompts, max_new_tokens=48, **sampling)
        assert [r.token_ids for r in got] == [r.token_ids for r in want]
        assert all(r.error is None and len(r.token_ids) == 48 for r in got)
        assert ahead.last_stats.preemptions > 0 and ahead.last_stats.launched_ahead > 0
        ahead.engine.cache.check_invariants()
        assert ahead.engine.cache.n_live() == 0
