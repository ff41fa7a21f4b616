"""A model whose layers need different caches, through the engine on the CPU twins of the kernels:
one attention layer keeps all keys, the other reads a window of them.  The cache manager then has
two groups of pages with a block table each; the windowed group gives pages back while a request
is still running, they are used again (the pool is too small otherwise), and every way of cutting
the requests gives the logits of the plain implementation."""

import random

import torch

import plain_llama
from torch_ops import TorchOps
from torchllms_b200.engine.model import Model
from torchllms_b200.engine.step import Engine, StepEntry
from torchllms_b200.parts.spec import LayerSpec, ModelSpec, RunEntry, part

DIM, H, KV, HD, HIDDEN, VOCAB, WINDOW, PAGE = 32, 4, 2, 8, 48, 97, 20, 4


def spec():
    rope = part("rope", head_dim=HD, theta=10000.0, scaling=None, pairing="interleaved")
    full = part("attention", dim=DIM, n_heads=H, n_kv_heads=KV, head_dim=HD, scale=HD ** -0.5, window=None, position=rope)
    near = part("attention", dim=DIM, n_heads=H, n_kv_heads=KV, head_dim=HD, scale=HD ** -0.5, window=WINDOW, position=rope)
    ffn = part("swiglu", dim=DIM, hidden=HIDDEN)
    norm = part("rmsnorm", dim=DIM, eps=1e-5)
    def blk(mixer):
        return part("prenorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                    mixer_prefix="mixer", ffn_prefix="ffn", mixer_norm_prefix="norm1", ffn_norm_prefix="norm2")
    layers = (LayerSpec("blocks.0", blk(full)), LayerSpec("blocks.1", blk(near)), LayerSpec("blocks.2", blk(near)))
    return ModelSpec(dim=DIM, vocab_size=VOCAB, max_positions=256, embedding_tensor="embed.weight", layers=layers,
                     run_order=(RunEntry(0), RunEntry(1), RunEntry(2)), final_norm=norm, final_norm_prefix="final_norm",
                     head_tensor="head.weight")


def plain_forward(w, tokens):
    """Whole sequence, no cache, from the plain functions (tests/plain_llama.py)."""
    S = len(tokens)
    cos, sin = plain_llama.rope_angles(plain_llama.rope_frequencies(HD, 10000.0, None), torch.arange(S))
    x = w["embed.weight"][torch.tensor(tokens)]
    for i, window in enumerate((None, WINDOW, WINDOW)):
        p = f"blocks.{i}"
        n = plain_llama.rms_norm(x, w[f"{p}.norm1.weight"], 1e-5)
        q = plain_llama.apply_rope((n @ w[f"{p}.mixer.wq.weight"].T).view(S, H, HD), cos, sin)
        k = plain_llama.apply_rope((n @ w[f"{p}.mixer.wk.weight"].T).view(S, KV, HD), cos, sin)
        v = (n @ w[f"{p}.mixer.wv.weight"].T).view(S, KV, HD)
        h = x + plain_llama.causal_attention(q, k, v, window=window) @ w[f"{p}.mixer.wo.weight"].T
        m = plain_llama.rms_norm(h, w[f"{p}.norm2.weight"], 1e-5)
        x = h + plain_llama.swiglu_ffn(m, w[f"{p}.ffn.w1.weight"], w[f"{p}.ffn.w2.weight"], w[f"{p}.ffn.w3.weight"])
    return plain_llama.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T


def loaded_model():
    model = Model(spec(), dtype=torch.float32, device="cpu", ops=TorchOps())
    g = torch.Generator().manual_seed(5)
    w = {name: (1 + 0.1 * torch.randn(e.shape, generator=g) if "norm" in name else torch.randn(e.shape, generator=g) * 0.3)
         for name, e in model.expected_tensors().items()}
    model.load(w)
    return model, w


def test_the_scheduler_admits_a_request_longer_than_the_window_groups_pool():
    """The window group has far fewer pages than a long request has tokens; it gives them back as
    the request grows, so the scheduler must take the request (and only refuse what the group that
    keeps every key cannot hold)."""
    from torchllms_b200.engine.scheduler import Request, Scheduler
    from torchllms_b200.sampling.sampler import Sampler
    model, w = loaded_model()
    engine = Engine(model, page_size=PAGE, pool_tokens=400, max_num_seqs=2, max_len=256, max_step_tokens=16)
    kinds = {g.need.kind: g for g in engine.cache.groups}
    window_tokens = kinds["window"].allocator.n_pages * PAGE
    rng = random.Random(3)
    prompts = [[rng.randrange(VOCAB) for _ in range(n)] for n in (150, 40)]
    assert window_tokens < 150 + 6                        # the old bound (smallest pool of any group) refused this
    sched = Scheduler(engine, Sampler(TorchOps(), "cpu"), max_num_batched_tokens=16, prefill_chunk=12)
    reqs = [Request(index=i, prompt=p, budget=6) for i, p in enumerate(prompts)]
    sched.run(reqs)
    for r, p in zip(reqs, prompts):
        assert r.error is None and len(r.generated) == 6
        seq = list(p)
        for tok in r.generated:                            # greedy against the plain forward
            assert tok == int(torch.argmax(plain_forward(w, seq)[-1]))
            seq.append(tok)
    engine.cache.check_invariants()
    assert engine.cache.n_live() == 0
    too_long = Request(index=2, prompt=[1] * 250, budget=10)     # 259 cached tokens: beyond max_len
    sched.add(too_long)
    assert too_long.finished and "at most 256" in too_long.error
    small = Engine(model, page_size=PAGE, pool_tokens=100, max_num_seqs=2, max_len=256, max_step_tokens=16)
    sched = Scheduler(small, Sampler(TorchOps(), "cpu"), max_num_batched_tokens=16, prefill_chunk=12)
    refused = Request(index=0, prompt=[1] * 120, budget=4)       # the group that keeps every key holds 100
    sched.add(refused)
    assert refused.finished and "at most 100" in refused.error


def test_full_and_windowed_layers_keep_pages_of_their_own():
    model, w = loaded_model()
    # The full group gets the pool it is asked for; the windowed group is sized by the manager for a
    # window and a step's tokens per request, far fewer pages than the requests' tokens need in all.
    engine = Engine(model, page_size=PAGE, pool_tokens=352, max_num_seqs=3, max_len=256, max_step_tokens=64)
    cache = engine.cache
    assert len(cache.groups) == 2
    kinds = {g.need.kind: g for g in cache.groups}
    assert kinds["full"].runs == [0] and kinds["window"].runs == [1, 2] and kinds["window"].need.window == WINDOW
    win = kinds["window"].index
    assert kinds["window"].allocator.n_pages * PAGE < 150 + 61 + 119 <= kinds["full"].allocator.n_pages * PAGE
    rng = random.Random(2)
    seqs = [[rng.randrange(VOCAB) for _ in range(n)] for n in (150, 61, 119)]
    want = [plain_forward(w, s) for s in seqs]
    handles = [engine.claim() for _ in seqs]
    fed = [0] * len(seqs)
    got = [[] for _ in seqs]
    sizes = [7, 1, 30, 2, 1, 13, 1, 1, 5, 22]
    most_window_pages = 0
    k = 0
    while any(f < len(s) for f, s in zip(fed, seqs)):
        entries, who = [], []
        for i, s in enumerate(seqs):
            if fed[i] < len(s) and (k + 2 * i) % 5 != 0:              # every request sits out a step now and then
                n = min(sizes[(k + 3 * i) % len(sizes)], len(s) - fed[i])
                entries.append(StepEntry(handles[i], s[fed[i]:fed[i] + n], list(range(n))))
                who.append((i, n))
                fed[i] += n
        k += 1
        if not entries:
            continue
        logits = engine.step(entries)
        cache.check_invariants()
        at = 0
        for i, n in who:
            got[i].append(logits[at:at + n])
            at += n
        for i, h in enumerate(handles):
            live = [p for p in cache.pages_of(h, win) if p >= 0]
            most_window_pages = max(most_window_pages, len(live))
            # about a window's worth of pages stays, however long the request has grown ...
            assert len(live) <= WINDOW // PAGE + 2
            # ... while the full group holds every page
            assert len([p for p in cache.pages_of(h, kinds["full"].index) if p >= 0]) == -(-fed[i] // PAGE)
    for i in range(len(seqs)):
        err = (torch.cat(got[i]) - want[i]).abs().max().item()
        assert err < 2e-4, (i, err)
    assert most_window_pages >= WINDOW // PAGE
    for h in handles:
        engine.release(h)
    cache.check_invariants()
    assert cache.n_live() == 0
    for grp in cache.groups:
        assert cache.free_pages(grp.index) == grp.allocator.n_pages
