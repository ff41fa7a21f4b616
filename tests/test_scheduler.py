"""The scheduler's decisions, on the CPU over the kernel twins and a tiny real model.

Restates the reference's driver tests for this engine (stop on any of several ids, budget
exhaustion, zero budgets, order of results, batched equals single:
torchllms/inference/test_prefix_cache_wiring.py:257-281, :379-549) and adds what the reference
does not have: token budgets, prompt portions, and pre-emption when pages run out."""

import pytest
import torch

from helpers import TINY, tiny_folder
from plain_llama import PlainModel
from torch_ops import TorchOps
from torchllms_b200.engine.loading import load_model
from torchllms_b200.engine.scheduler import Request, Scheduler
from torchllms_b200.engine.step import Engine
from torchllms_b200.inference import LLM
from torchllms_b200.sampling.sampler import Sampler, SamplingParams, row_key

OPS = TorchOps()
PROMPTS = [[1, 2, 3], [5], [7] * 40, [9, 8, 7, 6, 5, 4, 3, 2, 1] * 3, [11, 12] * 30, [400, 3, 77]]


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return tiny_folder(tmp_path_factory.mktemp("sched"), "A")


@pytest.fixture(scope="module")
def plain(folder):
    return PlainModel(folder)


def make_llm(folder, **kw):
    args = dict(device="cpu", precision="float32", max_len=128, max_bsz=4, page_size=16, ops=OPS,
                max_num_batched_tokens=48, prefill_chunk=24)
    args.update(kw)
    return LLM(folder, **args)


def make_scheduler(folder, *, pool_tokens, eos=(), **kw):
    _, _, model = load_model(folder, dtype="float32", device="cpu", ops=OPS)
    engine = Engine(model, page_size=16, pool_tokens=pool_tokens, max_num_seqs=kw.pop("max_num_seqs", 4),
                    max_len=128, max_step_tokens=kw.get("max_num_batched_tokens", 48))
    return Scheduler(engine, Sampler(OPS, "cpu"), eos_ids=eos, **kw)


def test_greedy_equals_plain_and_keeps_input_order(folder, plain):
    llm = make_llm(folder)
    got = llm.generate(prompt_token_ids=PROMPTS, max_new_tokens=6)
    assert [r.token_ids for r in got] == [plain.greedy(p, 6) for p in PROMPTS]
    assert all(r.stop_reason is None and r.error is None for r in got)
    llm.engine.cache.check_invariants()
    assert llm.engine.cache.n_live() == 0


def test_batched_equals_one_by_one(folder):
    llm = make_llm(folder)
    together = llm.generate(prompt_token_ids=PROMPTS, max_new_tokens=5, temperature=0.9, seed=3)
    alone = [llm.generate(prompt_token_ids=[p], max_new_tokens=5, temperature=0.9, seed=3)[0] for p in PROMPTS]
    # sampling noise is keyed by the request's place in its call, so compare place 0 with place 0
    assert together[0].token_ids == alone[0].token_ids
    greedy_together = llm.generate(prompt_token_ids=PROMPTS, max_new_tokens=5)
    greedy_alone = [llm.generate(prompt_token_ids=[p], max_new_tokens=5)[0] for p in PROMPTS]
    assert [r.token_ids for r in greedy_together] == [r.token_ids for r in greedy_alone]


def test_sampling_does_not_depend_on_cutting_or_batch_size(folder):
    a = make_llm(folder, max_num_batched_tokens=48, prefill_chunk=24, max_bsz=4)
    b = make_llm(folder, max_num_batched_tokens=7, prefill_chunk=3, max_bsz=2)
    c = make_llm(folder, max_num_batched_tokens=128, prefill_chunk=128, max_bsz=1)
    kw = dict(prompt_token_ids=PROMPTS, max_new_tokens=7, temperature=0.8, top_k=50, seed=7)
    ra, rb, rc = (x.generate(**kw) for x in (a, b, c))
    assert [r.token_ids for r in ra] == [r.token_ids for r in rb] == [r.token_ids for r in rc]
    other_seed = a.generate(**dict(kw, seed=8))
    assert [r.token_ids for r in other_seed] != [r.token_ids for r in ra]


def test_stop_on_any_of_keeps_the_stop_token(folder, plain):
    free = plain.greedy(PROMPTS[2], 8)
    stop_a, stop_b = free[3], free[5]
    llm = make_llm(folder, eos_ids=[stop_b, stop_a, 511])
    r = llm.generate(prompt_token_ids=[PROMPTS[2]], max_new_tokens=8)[0]
    first = min(free.index(stop_a), free.index(stop_b))
    assert r.token_ids == free[:first + 1] and r.stop_reason == free[first]


def test_budgets(folder, plain):
    llm = make_llm(folder, max_len=48)
    long_prompt = [3] * 45
    got = llm.generate(prompt_token_ids=[PROMPTS[0], long_prompt, [4] * 48, [4] * 60], max_new_tokens=10)
    assert len(got[0].token_ids) == 10 and got[0].stop_reason is None
    assert got[1].token_ids == plain.greedy(long_prompt, 3)          # min(max_len - prompt_len, max_new_tokens)
    assert got[2].token_ids == [] and got[3].token_ids == []          # no room at all: an empty result
    zero = llm.generate(prompt_token_ids=PROMPTS[:2], max_new_tokens=0)
    assert [r.token_ids for r in zero] == [[], []]
    with pytest.raises(ValueError):
        llm.generate(prompt_token_ids=[[]], max_new_tokens=2)
    with pytest.raises(ValueError):
        llm.generate(prompt_token_ids=PROMPTS, prompts=["x"])


def test_token_budget_and_portions_are_respected(folder):
    s = make_scheduler(folder, pool_tokens=512, max_num_batched_tokens=20, prefill_chunk=8)
    reqs = [Request(i, list(p), 4) for i, p in enumerate(PROMPTS)]
    s.run(reqs)
    for step in s.trace:
        assert sum(n for _, n in step) <= 20
        assert len(step) <= 4
    fed = {}
    for step in s.trace:
        for idx, n in step:
            fed.setdefault(idx, []).append(n)
    assert max(fed[2]) <= 8 and sum(fed[2]) == 40 + 3                 # 40 prompt tokens in portions, then 3 decodes
    assert fed[4][:3] == [8, 8, 8] or max(fed[4]) <= 8
    # decoding requests are never starved by prompt portions: once decoding, a request is in every step
    first_decode = {i: sum(1 for n in ns if n > 1) for i, ns in fed.items()}
    assert s.stats.decode_tokens == sum(len(r.generated) - 1 for r in reqs)
    assert s.stats.tokens == sum(len(p) for p in PROMPTS) + s.stats.decode_tokens


def test_requests_are_admitted_in_arrival_order(folder):
    s = make_scheduler(folder, pool_tokens=512, max_num_seqs=2, max_num_batched_tokens=64)
    reqs = [Request(i, [i + 1] * 5, 3) for i in range(5)]
    s.run(reqs)
    first_seen = []
    for step in s.trace:
        for idx, _ in step:
            if idx not in first_seen:
                first_seen.append(idx)
    assert first_seen == [0, 1, 2, 3, 4] and s.stats.max_running == 2


def test_preemption_when_pages_run_out_changes_no_token(folder, plain):
    prompts = [[7] * 30, [9, 8] * 14, [11] * 25]
    want = [plain.greedy(p, 24) for p in prompts]
    roomy = make_scheduler(folder, pool_tokens=512)
    tight = make_scheduler(folder, pool_tokens=112)                   # 7 pages: the three cannot all finish side by side
    for s in (roomy, tight):
        reqs = [Request(i, list(p), 24) for i, p in enumerate(prompts)]
        s.run(reqs)
        assert [r.generated for r in reqs] == want
        assert all(r.error is None for r in reqs)
        s.engine.cache.check_invariants()
        assert s.engine.cache.n_live() == 0 and s.engine.cache.free_pages() == s.engine.cache.groups[0].allocator.n_pages
    assert roomy.stats.preemptions == 0 and tight.stats.preemptions > 0
    # with a temperature too: the recomputed request draws the same noise
    a = make_scheduler(folder, pool_tokens=512)
    b = make_scheduler(folder, pool_tokens=112)
    outs = []
    for s in (a, b):
        reqs = [Request(i, list(p), 24, SamplingParams(0.8, None, 5)) for i, p in enumerate(prompts)]
        s.run(reqs)
        outs.append([r.generated for r in reqs])
    assert outs[0] == outs[1] and b.stats.preemptions > 0


def test_launching_the_next_step_ahead_changes_no_token(folder, plain):
    """The scheduler launches the next decode step before it has read this one's tokens.  Same
    tokens as without, through a stop token (a row computed in vain), a budget's end, a late
    arrival and a full pool; the cache is none the worse at any step."""
    prompts = [[7] * 30, [9, 8] * 14, [11] * 25, [5, 6, 7]]
    budgets = [24, 9, 17, 24]
    free = plain.greedy(prompts[1], 9)
    eos = (free[4],)                                                  # request 1 stops early on this
    runs = {}
    for ahead in (True, False):
        for pool in (512, 112):
            s = make_scheduler(folder, pool_tokens=pool, eos=eos, look_ahead=ahead)
            reqs = [Request(i, list(p), b, SamplingParams(0.7, 20, 3)) for i, (p, b) in enumerate(zip(prompts, budgets))]
            for r in reqs[:3]:
                s.add(r)
            for _ in range(6):
                s.step()
                s.engine.cache.check_invariants()
            s.add(reqs[3])                                            # arrives while the others decode
            while s.has_work():
                s.step()
                s.engine.cache.check_invariants()
            assert all(r.error is None and r.finished for r in reqs)
            assert s.engine.cache.n_live() == 0
            assert s.engine.cache.free_pages() == s.engine.cache.groups[0].allocator.n_pages
            runs[ahead, pool] = ([r.generated for r in reqs], s.trace, s.stats)
    for pool in (512, 112):
        assert runs[True, pool][0] == runs[False, pool][0]
        assert runs[True, pool][2].launched_ahead > 0 and runs[False, pool][2].launched_ahead == 0
        # the lost bets are the only extra work: one row for each request that stopped on a token
        assert runs[False, pool][2].tokens <= runs[True, pool][2].tokens <= runs[False, pool][2].tokens + len(prompts)
    assert runs[True, 112][2].preemptions > 0
    assert runs[True, 512][0] == runs[True, 112][0]


def test_a_request_that_can_never_fit_gets_an_error_not_a_hang(folder):
    s = make_scheduler(folder, pool_tokens=32)
    reqs = [Request(0, [1] * 40, 5), Request(1, [2] * 10, 5), Request(2, [3] * 20, 30)]
    s.run(reqs)
    assert reqs[0].error and reqs[0].generated == []
    assert reqs[1].error is None and len(reqs[1].generated) == 5
    assert reqs[2].error and "cached tokens" in reqs[2].error
    s.engine.cache.check_invariants()


def test_row_keys_are_distinct_and_stable():
    keys = {row_key(s, r, t) for s in range(3) for r in range(5) for t in range(7)}
    assert len(keys) == 3 * 5 * 7
    assert row_key(7, 2, 3) == row_key(7, 2, 3) and 0 <= row_key(1, 1, 1) < 2 ** 64


def test_chat_template_renders_llama3_turns():
    from torchllms_b200.inference.template import get_template
    t = get_template("llama3_instruct")
    text = t.render([{"role": "system", "content": " be brief "}, {"role": "user", "content": "hi"}])
    assert text == ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nbe brief<|eot_id|>"
                    "<|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>"
                    "<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert t.stop_token_ids == (128009,)
    with pytest.raises(ValueError):
        t.render([{"role": "wizard", "content": "x"}])


def test_chat_command_line_takes_the_references_options():
    """torchllms/inference/chat.py:15-46: the option names and defaults of the reference's chat."""
    from torchllms_b200.inference.chat import parse_args
    a = parse_args(["--ckpt_paths", "m1", "m2", "--template_config", "llama3_instruct", "--model_kwargs", '{"max_seq_len": 64}'])
    assert [str(p) for p in a.ckpt_paths] == ["m1", "m2"] and a.template_config == "llama3_instruct"
    assert a.max_new_tokens == 200 and a.temperature == 0.0 and a.device == "cuda" and a.precision is None
    assert a.model_kwargs == {"max_seq_len": 64}
    with pytest.raises(SystemExit):
        parse_args([])                      # a model folder is required


def test_progress_bar_counts_finished_requests_unless_disabled(folder, capsys):
    """``disable_tqdm`` as in the reference (torchllms/inference/llm.py:1081, :1126-1130): a bar on
    standard error unless disabled; here it counts requests, those without a budget included."""
    llm = make_llm(folder)
    capsys.readouterr()
    shown = llm.generate(prompt_token_ids=PROMPTS + [[4] * 128], max_new_tokens=3)      # the last one has no room
    err = capsys.readouterr().err
    n = len(PROMPTS) + 1
    assert f"{n}/{n}" in err and "generate" in err
    quiet = llm.generate(prompt_token_ids=PROMPTS + [[4] * 128], max_new_tokens=3, disable_tqdm=True)
    assert capsys.readouterr().err == ""
    assert [r.token_ids for r in shown] == [r.token_ids for r in quiet]


def test_entry_point_takes_the_references_arguments_in_their_order(folder):
    """torchllms/inference/llm.py:95-109: positional use must mean the same here."""
    import inspect
    names = list(inspect.signature(LLM.__init__).parameters)[1:13]
    assert names == ["ckpt_paths", "template_config", "eos_ids", "max_len", "max_bsz", "device", "precision",
                     "model_kwargs", "batched", "prefix_cache", "page_size", "kv_memory_gb"]
    names = list(inspect.signature(LLM.generate).parameters)[1:7]
    assert names == ["prompts", "conversations", "temperature", "max_new_tokens", "batch_size", "disable_tqdm"]
    with pytest.raises(ValueError, match="prefix cache"):
        make_llm(folder, prefix_cache=object())


@pytest.mark.parametrize("seed", range(24))
def test_random_arrivals_pools_and_budgets_change_no_token(folder, seed):
    """Random prompts, budgets, stop ids, pool sizes, token budgets, portion sizes, numbers of
    running requests and arrival times, with and without launching ahead: every request gets the
    tokens it gets when it runs alone in a roomy engine, the cache is sound after every step, and
    nothing is left behind.  A request that cannot fit the pool at all gets an error, not tokens."""
    import random
    rng = random.Random(1000 + seed)
    n = rng.randint(3, 7)
    prompts = [[rng.randrange(512) for _ in range(rng.choice([1, 2, 5, 17, 33, 60]))] for _ in range(n)]
    budgets = [rng.choice([0, 1, 2, 7, 12]) for _ in range(n)]
    sampling = SamplingParams(rng.choice([0.0, 0.8]), rng.choice([None, 20]), rng.randrange(100))
    alone = []
    for i, (p, b) in enumerate(zip(prompts, budgets)):
        s = make_scheduler(folder, pool_tokens=512)
        r = Request(i, list(p), b, sampling)
        s.run([r])
        alone.append(list(r.generated))
    # a stop id that some request meets on its way
    met = [t for g in alone for t in g[:-1]]
    eos = (rng.choice(met),) if met and rng.random() < 0.7 else ()
    def cut(g):
        for k, t in enumerate(g):
            if t in eos:
                return g[:k + 1]
        return g
    want = [cut(g) for g in alone]
    pool = rng.choice([48, 80, 112, 512])
    s = make_scheduler(folder, pool_tokens=pool, eos=eos, look_ahead=rng.random() < 0.5,
                       max_num_seqs=rng.randint(1, 4), max_num_batched_tokens=rng.choice([4, 9, 48]),
                       prefill_chunk=rng.choice([2, 5, 24]))
    reqs = [Request(i, list(p), b, sampling) for i, (p, b) in enumerate(zip(prompts, budgets))]
    late = list(reqs)
    rng.shuffle(late)
    first, late = late[:2], late[2:]
    for r in sorted(first, key=lambda r: r.index):
        s.add(r)
    steps = 0
    while s.has_work() or late:
        if late and (not s.has_work() or rng.random() < 0.3):
            s.add(late.pop())
        s.step()
        s.engine.cache.check_invariants()
        steps += 1
        assert steps < 2000, "the scheduler does not come to an end"
    for r, w, p, b in zip(reqs, want, prompts, budgets):
        assert r.finished
        need = len(p) + b - 1
        if b > 0 and -(-need // 16) * 16 > pool:
            assert r.error and r.generated == []
        else:
            assert r.error is None and r.generated == w, (r.index, r.generated, w)
            assert r.stop_reason == (w[-1] if w and w[-1] in eos else None)
    assert s.engine.cache.n_live() == 0
    assert s.engine.cache.free_pages() == s.engine.cache.groups[0].allocator.n_pages
