"""A mixer that is not attention, defined here, is registered, built and stepped through the
engine without a change to the framework's files: it keeps per-request state of fixed size (a
running sum and a count) in the cache manager's slots instead of pages.  The model that hosts it
also mixes it with attention layers, runs one layer twice and lets one run read another run's
cache, which the Llama spec never does."""

import pytest
import torch

import plain_llama
from torchllms_b200.engine.model import Model
from torchllms_b200.engine.step import Engine, StepEntry
from torchllms_b200.parts.base import MIXERS, Mixer, StateNeed, as_compute, register_mixer
from torchllms_b200.parts.spec import LayerSpec, ModelSpec, RunEntry, part
from torchllms_b200.weights.loader import ExpectedTensor

pytestmark = pytest.mark.gpu


class RunningMean(Mixer):
    """out[t] = W . mean(x[0..t]) of the request: needs the sum and count of earlier portions."""

    def __init__(self, env, *, dim):
        self.env, self.dim = env, dim
        self.w = None

    def state_need(self):
        return StateNeed((self.dim + 1,), torch.float32)

    def expected_tensors(self):
        return {"proj.weight": ExpectedTensor((self.dim, self.dim))}

    def load(self, tensors):
        self.w = as_compute(tensors["proj.weight"], self.env)

    def forward(self, x, ctx, cache):
        assert cache.k_pages is None and cache.state is not None
        out = torch.empty_like(x)
        starts = ctx.q_start.tolist()
        for i, slot in enumerate(ctx.slots):
            seg = x[starts[i]:starts[i + 1]].float()
            state = cache.state[slot]
            if ctx.fresh[i].item():
                assert float(state.abs().sum()) == 0.0          # the manager zeroed the slot on claim
            sums = state[:self.dim] + torch.cumsum(seg, 0)
            counts = state[self.dim] + torch.arange(1, seg.shape[0] + 1, device=x.device)
            out[starts[i]:starts[i + 1]] = (sums / counts[:, None]).to(x.dtype)
            state[:self.dim] = sums[-1]
            state[self.dim] = counts[-1]
        return self.env.ops.linear(out, self.w)


def toy_spec(dim, H, KV, hd, hidden, vocab):
    attn = part("attention", dim=dim, n_heads=H, n_kv_heads=KV, head_dim=hd, scale=hd ** -0.5, window=None,
                position=part("rope", head_dim=hd, theta=10000.0, scaling=None, pairing="interleaved"))
    mean = part("toy_running_mean", dim=dim)
    ffn = part("swiglu", dim=dim, hidden=hidden)
    norm = part("rmsnorm", dim=dim, eps=1e-5)
    blk = part("prenorm", mixer_prefix="mixer", ffn_prefix="ffn", mixer_norm_prefix="norm1", ffn_norm_prefix="norm2")
    layers = (LayerSpec("blocks.0", blk, attn, ffn, norm, norm), LayerSpec("blocks.1", blk, mean, ffn, norm, norm))
    # attention, running mean, the attention layer again with a cache of its own, and once more
    # reading the first run's cache
    order = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(0, cache_of=0), RunEntry(1))
    return ModelSpec(dim=dim, vocab_size=vocab, max_positions=256, embedding_tensor="embed.weight", layers=layers,
                     run_order=order, final_norm=norm, final_norm_prefix="final_norm", head_tensor="head.weight")


def plain_forward(w, tokens, dim, H, KV, hd):
    """Whole sequence, no cache: the same five runs written out with the plain functions."""
    cfg = {"n_heads": H, "n_kv_heads": KV, "head_dim": hd, "eps": 1e-5}
    S = len(tokens)
    cos, sin = plain_llama.rope_angles(plain_llama.rope_frequencies(hd, 10000.0, None), torch.arange(S))
    x = w["embed.weight"][torch.tensor(tokens)]
    kept = {}

    def attn_block(x, p, reuse=None):
        n = plain_llama.rms_norm(x, w[f"{p}.norm1.weight"], 1e-5)
        q = plain_llama.apply_rope((n @ w[f"{p}.mixer.wq.weight"].T).view(S, H, hd), cos, sin)
        if reuse is None:
            k = plain_llama.apply_rope((n @ w[f"{p}.mixer.wk.weight"].T).view(S, KV, hd), cos, sin)
            v = (n @ w[f"{p}.mixer.wv.weight"].T).view(S, KV, hd)
        else:
            k, v = reuse
        h = x + plain_llama.causal_attention(q, k, v) @ w[f"{p}.mixer.wo.weight"].T
        m = plain_llama.rms_norm(h, w[f"{p}.norm2.weight"], 1e-5)
        return h + plain_llama.swiglu_ffn(m, w[f"{p}.ffn.w1.weight"], w[f"{p}.ffn.w2.weight"], w[f"{p}.ffn.w3.weight"]), (k, v)

    def mean_block(x, p):
        n = plain_llama.rms_norm(x, w[f"{p}.norm1.weight"], 1e-5)
        means = torch.cumsum(n, 0) / torch.arange(1, S + 1)[:, None]
        h = x + means @ w[f"{p}.mixer.proj.weight"].T
        m = plain_llama.rms_norm(h, w[f"{p}.norm2.weight"], 1e-5)
        return h + plain_llama.swiglu_ffn(m, w[f"{p}.ffn.w1.weight"], w[f"{p}.ffn.w2.weight"], w[f"{p}.ffn.w3.weight"])

    x, first_cache = attn_block(x, "blocks.0")
    x = mean_block(x, "blocks.1")
    x, _ = attn_block(x, "blocks.0")
    x, _ = attn_block(x, "blocks.0", reuse=first_cache)
    x = mean_block(x, "blocks.1")
    return plain_llama.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from torchllms_b200.kernels import get_ops
    register_mixer("toy_running_mean")(RunningMean)
    try:
        dim, H, KV, hd, hidden, vocab = 48, 3, 1, 16, 80, 131
        spec = toy_spec(dim, H, KV, hd, hidden, vocab)
        model = Model(spec, dtype=torch.float32, device="cuda", ops=get_ops())
        g = torch.Generator().manual_seed(3)
        w = {name: (1 + 0.1 * torch.randn(e.shape, generator=g) if "norm" in name else torch.randn(e.shape, generator=g) * 0.12)
             for name, e in model.expected_tensors().items()}
        assert "blocks.1.mixer.proj.weight" in w and "blocks.0.mixer.wq.weight" in w
        model.load(w)
        needs = model.run_needs()
        assert [n[0] is not None for n in needs] == [True, False, True, True, False]
        assert [n[1] is not None for n in needs] == [False, True, False, False, True] and needs[3][2] == 0
        engine = Engine(model, page_size=8, pool_tokens=256, max_num_seqs=3, max_len=256, max_step_tokens=128)
        assert len(engine.cache.groups) == 1 and engine.cache.groups[0].runs == [0, 2]     # run 3 borrows run 0's pages
        assert engine.cache.state[1].shape == (3, dim + 1) and engine.cache.state[4] is not engine.cache.state[1]
        gen = torch.Generator().manual_seed(4)
        seqs = [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in (37, 5, 60)]
        want = [plain_forward(w, s, dim, H, KV, hd) for s in seqs]
        handles = [engine.claim() for _ in seqs]
        fed = [0, 0, 0]
        got = [[] for _ in seqs]
        sizes = [5, 2, 11, 1, 7, 3, 19, 2]
        k = 0
        while any(f < len(s) for f, s in zip(fed, seqs)):
            entries, who = [], []
            for i, s in enumerate(seqs):
                if fed[i] < len(s) and (k + i) % 4 != 0:              # every request sits out a step now and then
                    n = min(sizes[(k + i) % len(sizes)], len(s) - fed[i])
                    entries.append(StepEntry(handles[i], s[fed[i]:fed[i] + n], list(range(n))))
                    who.append((i, n))
                    fed[i] += n
            k += 1
            if not entries:
                continue
            logits = engine.step(entries).cpu()
            at = 0
            for i, n in who:
                got[i].append(logits[at:at + n])
                at += n
        for i in range(len(seqs)):
            err = (torch.cat(got[i]) - want[i]).abs().max().item()
            assert err < 1e-4, (i, err)
        # a released slot is zeroed for the next request
        engine.release(handles[1])
        h = engine.claim()
        again = engine.step([StepEntry(h, seqs[1], list(range(len(seqs[1]))))]).cpu()
        assert (again - want[1]).abs().max().item() < 1e-4
        engine.cache.check_invariants()
    finally:
        MIXERS.unregister("toy_running_mean")
