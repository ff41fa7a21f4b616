"""The engine's host side (cache, step function, replay) on the CPU over the plain PyTorch twins
of the kernels: every way of cutting and batching must reproduce the plain implementation."""

import random

import numpy as np
import pytest
import torch

import traces
from helpers import TINY, tiny_folder
from plain_llama import PlainModel
from torch_ops import TorchOps
from torchllms_b200.engine.replay import Replayer

LENGTHS = {"A": [1, 7, 33, 64, 97, 50, 120, 20, 3, 70], "B": [2, 5, 17, 40, 100, 65, 129, 30, 90],
           "D": [3, 50, 131, 64, 17, 90, 2, 120, 77, 101]}
# The plain implementation itself sits about 1.3e-5 from a float64 evaluation of these
# (deliberately peaked) models, so float32 paths that sum in another order differ by a few 1e-5.
ATOL = 1e-4


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in ("A", "B", "D"):                 # the third configuration is for GPU kernels
        cfg, seed, page = TINY[name]
        folder = tiny_folder(tmp_path_factory.mktemp(name), name)
        rng = random.Random(seed)
        reqs = {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}
        plain = PlainModel(folder)
        out[name] = (folder, page, reqs, {rid: plain.logits(t).numpy() for rid, t in reqs.items()})
    return out


@pytest.mark.parametrize("name", ["A", "B", "D"])
@pytest.mark.parametrize("mode", ["whole", "tail_one_by_one", "portions", "mixed"])
def test_cuts_agree_with_plain(setups, name, mode):
    folder, page, reqs, ref = setups[name]
    steps, places, peak = getattr(traces, mode)(reqs)
    rp = Replayer(folder, "float32", peak, page_size=page, device="cpu", ops=TorchOps())
    for s in steps:
        got = rp.run_step(s)
        rp.engine.cache.check_invariants()
        if s["step"] in places:
            want = np.stack([ref[rid][pos] for rid, pos in places[s["step"]]])
            assert np.abs(got - want).max() < ATOL, (mode, s["step"])
        else:
            assert got is None
    assert rp.engine.cache.n_live() == 0
    assert rp.engine.cache.free_pages() == rp.engine.cache.groups[0].allocator.n_pages
    if mode == "mixed":
        # the pool was sized to the peak, so pages must have been used again
        assert sum(-(-len(t) // page) for t in reqs.values()) > rp.engine.cache.groups[0].allocator.n_pages


def test_step_rejects_bad_input(setups):
    from torchllms_b200.engine.step import StepEntry, StepError
    from torchllms_b200.cache.manager import OutOfPages
    folder, page, reqs, _ = setups["A"]
    rp = Replayer(folder, "float32", 64, page_size=page, device="cpu", ops=TorchOps())
    eng = rp.engine
    h = eng.claim()
    with pytest.raises(StepError):
        eng.step([StepEntry(h, [512])])                  # outside the vocabulary
    with pytest.raises(StepError):
        eng.step([StepEntry(h, [])])
    with pytest.raises(StepError):
        eng.step([StepEntry(h, [1, 2], want=[2])])
    eng.step([StepEntry(h, list(range(60)))])
    with pytest.raises(OutOfPages):
        eng.step([StepEntry(h, list(range(10)))])        # 70 tokens do not fit 64
    assert eng.cache.length(h) == 60                     # nothing changed
    eng.cache.check_invariants()


def test_a_step_in_two_halves_and_a_step_called_off(setups):
    """``step`` is ``prepare`` (cache growth and index data, no token values) plus ``run_prepared``
    (token ids from a host list or from a device tensor with a row index).  A prepared step that is
    called off, or whose tokens turn out bad, leaves the cache as it was."""
    from torchllms_b200.engine.step import StepEntry, StepError
    folder, page, reqs, ref = setups["B"]
    rp = Replayer(folder, "float32", 256, page_size=page, device="cpu", ops=TorchOps())
    eng = rp.engine
    toks = reqs["r3"]                                    # 40 tokens
    a, b = eng.claim(), eng.claim()
    eng.step([StepEntry(a, toks[:30], []), StepEntry(b, toks[:7], [])])
    before = (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages())
    called_off = eng.prepare([(a, 5, None), (b, 20, [0])])
    assert (eng.cache.length(a), eng.cache.length(b)) == (35, 27)
    eng.discard(called_off)
    assert (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages()) == before
    bad = eng.prepare([(a, 2, None)])
    with pytest.raises(StepError):
        eng.run_prepared(bad, [1, 100000])               # outside the vocabulary: rolled back
    assert (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages()) == before
    # the same step from a host list and from a "device" tensor gathered by rows
    want = eng.step([StepEntry(a, toks[30:31], [0]), StepEntry(b, toks[7:8], [0])]).clone()
    eng.cache.truncate(a, 30)
    eng.cache.truncate(b, 7)
    prepared = eng.prepare([(a, 1, [0]), (b, 1, [0])])
    pool = torch.tensor([toks[7], 3, toks[30]], dtype=torch.int32)
    got = eng.run_prepared(prepared, pool, rows=[2, 0])
    assert torch.equal(got, want)
    assert np.abs(got[0].numpy() - ref["r3"][30]).max() < ATOL
    with pytest.raises(StepError):
        eng.run_prepared(eng.prepare([(a, 1, None)]), pool, rows=[3])    # no such row
    eng.cache.check_invariants()


def test_the_context_bound_that_steps_of_short_portions_plan_for(setups):
    """Few requests plan for the power of two that holds their longest context (at least 1,024, at
    most the engine's limit), sixteen or more for the limit itself."""
    folder, page, _, _ = setups["A"]
    eng = Replayer(folder, "float32", 64, page_size=page, device="cpu", ops=TorchOps()).engine
    assert eng.max_len == 128
    assert eng.kv_bound(1, 1) == eng.kv_bound(128, 3) == 128 and eng.kv_bounds(1) == [128]
    eng.max_len = 5000                                    # (the arithmetic only: no step runs with it)
    assert [eng.kv_bound(n, 2) for n in (1, 1024, 1025, 2048, 2049, 4096, 4097, 5000)] == \
           [1024, 1024, 2048, 2048, 4096, 4096, 5000, 5000]
    assert eng.kv_bounds(15) == [1024, 2048, 4096, 5000]
    assert eng.kv_bound(7, 16) == 5000 and eng.kv_bounds(16) == [5000] and eng.kv_bounds(64) == [5000]


def test_one_token_entries_are_moved_to_the_head_of_the_batch_and_rows_keep_the_callers_order(setups):
    """A caller may hand decode tokens and prompt portions in any order: inside the batch the
    one-token entries stand first (the mixer sends them to the decode kernel), the returned rows
    follow the caller's entries."""
    from torchllms_b200.engine.step import StepEntry
    folder, page, reqs, ref = setups["B"]
    rp = Replayer(folder, "float32", 512, page_size=page, device="cpu", ops=TorchOps())
    eng = rp.engine
    ids = ["r4", "r2", "r5", "r3"]                       # 100, 17, 65, 40 tokens
    hs = {r: eng.claim() for r in ids}
    eng.step([StepEntry(hs["r2"], reqs["r2"][:10], []), StepEntry(hs["r3"], reqs["r3"][:30], [])])
    # portion, decode token, portion, decode token
    entries = [StepEntry(hs["r4"], reqs["r4"][:20], [0, 19]), StepEntry(hs["r2"], reqs["r2"][10:11], [0]),
               StepEntry(hs["r5"], reqs["r5"][:33], [5]), StepEntry(hs["r3"], reqs["r3"][30:31], [0])]
    prepared = eng.prepare([(e.handle, len(e.tokens), e.want) for e in entries])
    assert prepared.order == [1, 3, 0, 2] and prepared.q_lens == [1, 1, 20, 33]
    got = eng.run_prepared(prepared, [t for e in entries for t in e.tokens]).numpy()
    want = np.stack([ref["r4"][0], ref["r4"][19], ref["r2"][10], ref["r5"][5], ref["r3"][30]])
    assert np.abs(got - want).max() < ATOL
    # the same with the ids taken from a tensor by rows (the way the scheduler feeds a step ahead)
    entries = [StepEntry(hs["r4"], reqs["r4"][20:23], [2]), StepEntry(hs["r2"], reqs["r2"][11:12], [0])]
    flat = [t for e in entries for t in e.tokens]
    pool = torch.tensor([7] + flat[::-1], dtype=torch.int32)
    prepared = eng.prepare([(e.handle, len(e.tokens), e.want) for e in entries])
    assert prepared.order == [1, 0]
    got = eng.run_prepared(prepared, pool, rows=[4, 3, 2, 1]).numpy()
    assert np.abs(got - np.stack([ref["r4"][22], ref["r2"][11]])).max() < ATOL
    eng.cache.check_invariants()


def test_a_failed_prepare_leaves_the_cache_as_it_was(setups, monkeypatch):
    from torchllms_b200.engine.step import StepError
    folder, page, reqs, _ = setups["A"]
    eng = Replayer(folder, "float32", 128, page_size=page, device="cpu", ops=TorchOps()).engine
    a, b = eng.claim(), eng.claim()
    eng.prepare([(a, 20, []), (b, 3, [])])
    before = (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages())
    with pytest.raises(StepError, match="twice"):
        eng.prepare([(a, 2, [1, 1])])                     # checked before anything grows
    assert (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages()) == before
    monkeypatch.setattr(eng.cache, "block_table_rows", lambda *a, **k: (_ for _ in ()).throw(RuntimeError("boom")))
    with pytest.raises(RuntimeError, match="boom"):
        eng.prepare([(a, 30, None), (b, 1, None)])        # fails after the cache has grown: rolled back
    assert (eng.cache.length(a), eng.cache.length(b), eng.cache.free_pages()) == before
    eng.cache.check_invariants()


def test_an_engine_shorter_than_the_models_position_table_runs_mixed_steps(setups):
    """The block table is as wide as the engine's limit, not the model's: every bound a step plans
    for must come from the engine."""
    from torchllms_b200.engine.loading import load_model
    from torchllms_b200.engine.step import Engine, StepEntry
    folder, page, reqs, ref = setups["B"]
    _, cfg, model = load_model(folder, dtype="float32", device="cpu", ops=TorchOps())
    assert model.max_positions == 256
    eng = Engine(model, page_size=page, pool_tokens=192, max_num_seqs=3, max_len=96, max_step_tokens=64)
    assert eng.cache.max_blocks * page == 96
    a, b = eng.claim(), eng.claim()
    eng.step([StepEntry(a, reqs["r3"][:30], [])])
    got = eng.step([StepEntry(a, reqs["r3"][30:31], [0]), StepEntry(b, reqs["r5"][:40], [39])]).numpy()   # decode beside a portion
    assert np.abs(got - np.stack([ref["r3"][30], ref["r5"][39]])).max() < ATOL
    got = eng.step([StepEntry(b, reqs["r5"][40:41], [0]), StepEntry(a, reqs["r3"][31:32], [0])]).numpy()
    assert np.abs(got - np.stack([ref["r5"][40], ref["r3"][31]])).max() < ATOL


def test_debug_mode_checks_every_index_array_on_the_host(setups):
    from torchllms_b200.engine.step import StepError
    folder, page, reqs, ref = setups["A"]
    eng = Replayer(folder, "float32", 128, page_size=page, device="cpu", ops=TorchOps()).engine
    eng.debug = True
    a, b = eng.claim(), eng.claim()
    p = eng.prepare([(a, 20, [3]), (b, 1, None)])         # a sound step passes
    eng.run_prepared(p, list(range(21)))
    n_pages = eng.cache.groups[0].allocator.n_pages
    for name, index, value, what in (("block_table0", 1, n_pages, "block_table0"), ("slot_mapping0", 2, n_pages * page, "slot_mapping0"),
                                      ("want_rows", 0, 99, "want_rows"), ("positions", 0, -1, "positions"),
                                      ("kv_len", 1, 0, "kv_len"), ("q_start", 1, 0, "q_start")):
        eng.prepare([(a, 4, [0]), (b, 2, [1])])
        eng._buf.host_view(name)[index] = value
        with pytest.raises(StepError, match=what):
            eng._check_packed(6, 2, 2)
        eng.cache.truncate(a, 20)
        eng.cache.truncate(b, 1)
