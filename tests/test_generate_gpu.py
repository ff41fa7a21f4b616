"""Greedy generation through the Python entry point on the GPU against the plain implementation."""

import pytest
import torch

from helpers import TINY, tiny_folder
from plain_llama import PlainModel, to_bfloat16_and_back

pytestmark = pytest.mark.gpu

PROMPTS = {"A": [[1, 2, 3], [5], [7] * 40, list(range(100, 164)), [11, 12] * 30],
           "B": [[999, 0], [5, 17, 3, 41, 8], list(range(200, 300)), [3] * 17, [900 - i for i in range(200)]]}


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_float32_matches_plain_token_for_token(tmp_path, name):
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY[name]
    folder = tiny_folder(tmp_path, name)
    llm = LLM(folder, precision="float32", max_len=cfg["max_position_embeddings"], max_bsz=3, page_size=page,
              max_num_batched_tokens=64, prefill_chunk=24)
    got = llm.generate(prompt_token_ids=PROMPTS[name], max_new_tokens=16)
    plain = PlainModel(folder)
    for p, r in zip(PROMPTS[name], got):
        assert r.token_ids == plain.greedy(p, 16), p
    llm.engine.cache.check_invariants()
    assert llm.engine.cache.n_live() == 0
    # tight pool: the same tokens although requests are pre-empted and recomputed
    per_token = cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * 4
    pool_tokens = max(len(p) for p in PROMPTS[name]) + 16 + 2 * page
    small = LLM(folder, precision="float32", max_len=cfg["max_position_embeddings"], max_bsz=3, page_size=page,
                kv_memory_gb=pool_tokens * per_token / 2 ** 30, max_num_batched_tokens=64, prefill_chunk=24)
    assert small.engine.cache.groups[0].allocator.n_pages == pool_tokens // page
    assert [r.token_ids for r in small.generate(prompt_token_ids=PROMPTS[name], max_new_tokens=16)] == [r.token_ids for r in got]
    assert small.last_stats.preemptions > 0 or small.last_stats.max_running < 3


# how far apart the two best logits must be before bfloat16 has to agree on the winner: twice what
# the replay tests allow these models (a quarter of what bfloat16 storage moves their logits)
MARGIN = {"A": 0.03, "B": 0.12}


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_bfloat16_follows_plain_while_the_margin_is_clear(tmp_path, name):
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY[name]
    folder = tiny_folder(tmp_path, name, dtype=torch.bfloat16)
    llm = LLM(folder, precision="bfloat16", max_len=cfg["max_position_embeddings"], max_bsz=4, page_size=page,
              max_num_batched_tokens=64, prefill_chunk=24)
    got = llm.generate(prompt_token_ids=PROMPTS[name], max_new_tokens=12)
    plain = PlainModel(folder)
    checked = 0
    for p, r in zip(PROMPTS[name], got):
        seq = list(p)
        for tok in r.token_ids:                        # follow the engine's tokens, judge each one
            logits = plain.logits(seq, stored=to_bfloat16_and_back)[-1]
            top = torch.topk(logits, 2)
            if float(top.values[0] - top.values[1]) >= MARGIN[name]:
                assert tok == int(top.indices[0]), (p, len(seq))
                checked += 1
            else:                                      # a near tie: either of the two is a fair answer
                assert tok in top.indices.tolist() or float(top.values[0] - logits[tok]) < MARGIN[name], (p, len(seq))
            seq.append(tok)
    assert checked >= 15


def test_temperature_sampling_is_reproducible_and_seeded(tmp_path):
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY["A"]
    folder = tiny_folder(tmp_path, "A")
    a = LLM(folder, precision="float32", max_len=128, max_bsz=4, page_size=page, max_num_batched_tokens=64, prefill_chunk=24)
    b = LLM(folder, precision="float32", max_len=128, max_bsz=2, page_size=page, max_num_batched_tokens=9, prefill_chunk=4)
    kw = dict(prompt_token_ids=PROMPTS["A"], max_new_tokens=10, temperature=0.8, seed=7)
    ra, rb = a.generate(**kw), b.generate(**kw)
    assert [r.token_ids for r in ra] == [r.token_ids for r in rb]
    assert [r.token_ids for r in a.generate(**dict(kw, seed=8))] != [r.token_ids for r in ra]
    top1 = a.generate(prompt_token_ids=PROMPTS["A"], max_new_tokens=10, temperature=1.5, top_k=1)
    greedy = a.generate(prompt_token_ids=PROMPTS["A"], max_new_tokens=10)
    assert [r.token_ids for r in top1] == [r.token_ids for r in greedy]


@pytest.mark.parametrize("precision", ["float32", "bfloat16"])
def test_launching_ahead_gives_the_same_tokens_on_the_device(tmp_path, precision):
    """The scheduler feeds a decode step from the sampler's output on the device before the host
    has read it.  Same tokens as the step-by-step way, greedy and with a temperature, when requests
    of different budgets leave one by one (the device-side gather) and when one stops on a token."""
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY["B"]
    folder = tiny_folder(tmp_path, "B")
    prompts = PROMPTS["B"]
    kw = dict(precision=precision, max_len=256, max_bsz=4, page_size=page, max_num_batched_tokens=64, prefill_chunk=24)
    plain_way = LLM(folder, look_ahead=False, **kw)
    for sampling in (dict(), dict(temperature=0.9, top_k=12, seed=5), dict(temperature=0.7, seed=6)):
        want = plain_way.generate(prompt_token_ids=prompts, max_new_tokens=40, **sampling)
        stop = want[0].token_ids[17]
        ahead = LLM(folder, look_ahead=True, eos_ids=[stop], **kw)
        stepwise = LLM(folder, look_ahead=False, eos_ids=[stop], **kw)
        got, ref = (x.generate(prompt_token_ids=prompts, max_new_tokens=40, **sampling) for x in (ahead, stepwise))
        assert [r.token_ids for r in got] == [r.token_ids for r in ref]
        assert [r.stop_reason for r in got] == [r.stop_reason for r in ref] and got[0].stop_reason == stop
        assert ahead.last_stats.launched_ahead > 10 and stepwise.last_stats.launched_ahead == 0
        ahead.engine.cache.check_invariants()
        assert ahead.engine.cache.n_live() == 0


def test_cache_pool_as_a_share_of_free_memory(tmp_path):
    """Three ways to size the cache: requests x length (default), GiB, or a share of what the device
    has free once the weights are on it."""
    from torchllms_b200.inference import LLM
    cfg, _, page = TINY["A"]
    folder = tiny_folder(tmp_path, "A")
    kw = dict(precision="float32", max_len=128, max_bsz=2, page_size=page)
    by_count = LLM(folder, **kw)
    assert by_count.engine.cache.groups[0].allocator.n_pages * page == 2 * 128
    free_before, _ = torch.cuda.mem_get_info()
    by_share = LLM(folder, kv_memory_fraction=0.001, **kw)
    per_token = 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 4
    tokens = by_share.engine.cache.groups[0].allocator.n_pages * page
    assert 0.5 * 0.001 * free_before / per_token < tokens <= 0.001 * free_before / per_token + page
    out = by_share.generate(prompt_token_ids=PROMPTS["A"][:2], max_new_tokens=4)
    assert [r.token_ids for r in out] == [r.token_ids for r in by_count.generate(prompt_token_ids=PROMPTS["A"][:2], max_new_tokens=4)]
    with pytest.raises(ValueError):
        LLM(folder, kv_memory_fraction=0.5, kv_memory_gb=1.0, **kw)
    with pytest.raises(ValueError):
        LLM(folder, kv_memory_fraction=1.5, **kw)


def test_chat_command_line_in_token_ids(tmp_path, monkeypatch, capsys):
    """The chat command line on a folder without a tokenizer: lines of token ids in, generated ids out,
    the history carried from turn to turn, ``!!reset`` starting over, end of input ending the chat."""
    from torchllms_b200.inference import chat
    cfg, _, _page = TINY["A"]
    folder = tiny_folder(tmp_path, "A")
    lines = iter(["5 17 3", "not ids", "8 9", "!!reset", "5 17 3"])

    def fake_input(prompt=""):
        try:
            return next(lines)
        except StopIteration:
            raise EOFError
    monkeypatch.setattr("builtins.input", fake_input)
    chat.main(["--ckpt_paths", str(folder), "--precision", "float32", "--max_new_tokens", "6",
               "--max_len", str(cfg["max_position_embeddings"])])
    said = [l[len("[assistant]: "):] for l in capsys.readouterr().out.splitlines() if l.startswith("[assistant]: ")]
    assert len(said) == 3
    plain = PlainModel(folder)
    first = plain.greedy([5, 17, 3], 6)
    assert said[0] == " ".join(map(str, first))
    assert said[1] == " ".join(map(str, plain.greedy([5, 17, 3] + first + [8, 9], 6)))     # the history is carried
    assert said[2] == said[0]                                                               # and dropped by !!reset
