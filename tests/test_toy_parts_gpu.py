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
    def blk(mixer):
        return part("prenorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=norm,
                    mixer_prefix="mixer", ffn_prefix="ffn", mixer_norm_prefix="norm1", ffn_norm_prefix="norm2")
    layers = (LayerSpec("blocks.0", blk(attn)), LayerSpec("blocks.1", blk(mean)))
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


# --------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, both defined here.

from torchllms_b200.parts.base import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding,  # noqa: E402
                                       register_feed_forward, register_position_encoding)


class RoutedFFN(FeedForward):
    """Top-1 routing over small experts: out = gate * W_out[e] relu(W_in[e] x), e = argmax(router x).
    Router logits and the softmax over them are float32."""

    def __init__(self, env, *, dim, hidden, n_experts):
        self.env, self.dim, self.hidden, self.n_experts = env, dim, hidden, n_experts

    def expected_tensors(self):
        out = {"router.weight": ExpectedTensor((self.n_experts, self.dim))}
        for e in range(self.n_experts):
            out[f"experts.{e}.w_in.weight"] = ExpectedTensor((self.hidden, self.dim))
            out[f"experts.{e}.w_out.weight"] = ExpectedTensor((self.dim, self.hidden))
        return out

    def load(self, tensors):
        self.router = tensors["router.weight"].to(self.env.device, torch.float32)
        self.w_in = [as_compute(tensors[f"experts.{e}.w_in.weight"], self.env) for e in range(self.n_experts)]
        self.w_out = [as_compute(tensors[f"experts.{e}.w_out.weight"], self.env) for e in range(self.n_experts)]

    def forward(self, x, ctx):
        probs = torch.softmax(x.float() @ self.router.t(), -1)
        gate, choice = probs.max(-1)
        out = torch.zeros_like(x)
        for e in range(self.n_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h = torch.relu(self.env.ops.linear(x[rows].contiguous(), self.w_in[e]))
                out[rows] = (self.env.ops.linear(h, self.w_out[e]).float() * gate[rows, None]).to(x.dtype)
        return out


class LearnedOffsets(PositionEncoding):
    """No rotation: a learned vector per position is added to q and k (float32 sum), v is stored as it is."""

    def __init__(self, env, *, head_dim, max_positions):
        self.env, self.head_dim, self.max_positions = env, head_dim, max_positions

    def expected_tensors(self):
        return {"offsets.weight": ExpectedTensor((self.max_positions, self.head_dim))}

    def load(self, tensors):
        self.offsets = tensors["offsets.weight"].to(self.env.device, torch.float32)
        # an identity table lets the fused kernel do the split and the cache write without rotating
        ident = torch.zeros(self.max_positions, self.head_dim // 2, 2)
        ident[..., 0] = 1.0
        self.identity = ident.to(self.env.device)

    def encode_and_store(self, qkv, ctx, cache, n_heads, n_kv_heads, head_dim):
        T = qkv.shape[0]
        x = qkv.float().view(T, n_heads + 2 * n_kv_heads, head_dim).clone()
        x[:, : n_heads + n_kv_heads] += self.offsets[ctx.positions.long()][:, None, :]
        shifted = x.view(T, -1).to(qkv.dtype)
        return self.env.ops.rope_kv_write(
            shifted, ctx.positions, self.identity, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
            interleaved=True, k_pages=cache.k_pages if cache.writes else None,
            v_pages=cache.v_pages if cache.writes else None, slot_mapping=cache.slot_mapping, page_size=cache.page_size)


def test_toy_routed_feed_forward_and_other_position_encodings():
    from torchllms_b200.kernels import get_ops
    register_feed_forward("toy_routed")(RoutedFFN)
    register_position_encoding("toy_learned_offsets")(LearnedOffsets)
    try:
        dim, H, KV, hd, vocab, E = 64, 4, 2, 16, 97, 3
        norm = part("rmsnorm", dim=dim, eps=1e-5)
        def blk(mixer, feed_forward):
            return part("prenorm", mixer=mixer, feed_forward=feed_forward, mixer_norm=norm, ffn_norm=norm,
                        mixer_prefix="mixer", ffn_prefix="ffn", mixer_norm_prefix="norm1", ffn_norm_prefix="norm2")
        attn_learned = part("attention", dim=dim, n_heads=H, n_kv_heads=KV, head_dim=hd, scale=hd ** -0.5, window=None,
                            position=part("toy_learned_offsets", head_dim=hd, max_positions=128))
        attn_half = part("attention", dim=dim, n_heads=H, n_kv_heads=KV, head_dim=hd, scale=hd ** -0.5, window=None,
                         position=part("rope", head_dim=hd, theta=100.0, scaling=None, pairing="half"))
        routed = part("toy_routed", dim=dim, hidden=40, n_experts=E)
        dense = part("swiglu", dim=dim, hidden=72)
        spec = ModelSpec(dim=dim, vocab_size=vocab, max_positions=128, embedding_tensor="embed.weight",
                         layers=(LayerSpec("l0", blk(attn_learned, routed)), LayerSpec("l1", blk(attn_half, dense))),
                         run_order=(RunEntry(0), RunEntry(1)), final_norm=norm, final_norm_prefix="final_norm",
                         head_tensor="head.weight")
        model = Model(spec, dtype=torch.float32, device="cuda", ops=get_ops())
        assert not model.graph_safe          # parts that read back on the host keep the engine off CUDA graphs
        g = torch.Generator().manual_seed(11)
        w = {n: (1 + 0.1 * torch.randn(e.shape, generator=g) if "norm" in n else torch.randn(e.shape, generator=g) * 0.15)
             for n, e in model.expected_tensors().items()}
        # a position encoding's tensors live under the mixer that owns it
        assert "l0.mixer.position.offsets.weight" in w and "l0.ffn.experts.2.w_out.weight" in w
        model.load(w)
        engine = Engine(model, page_size=8, pool_tokens=128, max_num_seqs=2, max_len=128, max_step_tokens=64)
        toks = torch.randint(0, vocab, (50,), generator=g).tolist()

        # ---- the same model written out plainly, whole sequence, no cache
        S = len(toks)
        x = w["embed.weight"][torch.tensor(toks)]
        offsets = w["l0.mixer.position.offsets.weight"]

        def attend(x, p, encode):
            n = plain_llama.rms_norm(x, w[f"{p}.norm1.weight"], 1e-5)
            q = (n @ w[f"{p}.mixer.wq.weight"].T).view(S, H, hd)
            k = (n @ w[f"{p}.mixer.wk.weight"].T).view(S, KV, hd)
            v = (n @ w[f"{p}.mixer.wv.weight"].T).view(S, KV, hd)
            q, k = encode(q), encode(k)
            return x + plain_llama.causal_attention(q, k, v) @ w[f"{p}.mixer.wo.weight"].T

        def half_rope(t):
            inv = plain_llama.rope_frequencies(hd, 100.0, None)
            cos, sin = plain_llama.rope_angles(inv, torch.arange(S))
            a, b = t[..., : hd // 2], t[..., hd // 2:]
            c, s_ = cos[:, None, :], sin[:, None, :]
            return torch.cat([a * c - b * s_, b * c + a * s_], -1)

        h = attend(x, "l0", lambda t: t + offsets[:S, None, :])
        n = plain_llama.rms_norm(h, w["l0.norm2.weight"], 1e-5)
        probs = torch.softmax(n @ w["l0.ffn.router.weight"].T, -1)
        gate, choice = probs.max(-1)
        ff = torch.zeros_like(n)
        for t in range(S):
            e = int(choice[t])
            ff[t] = gate[t] * (torch.relu(n[t] @ w[f"l0.ffn.experts.{e}.w_in.weight"].T) @ w[f"l0.ffn.experts.{e}.w_out.weight"].T)
        h = h + ff
        h = attend(h, "l1", half_rope)
        m = plain_llama.rms_norm(h, w["l1.norm2.weight"], 1e-5)
        h = h + plain_llama.swiglu_ffn(m, w["l1.ffn.w1.weight"], w["l1.ffn.w2.weight"], w["l1.ffn.w3.weight"])
        want = plain_llama.rms_norm(h, w["final_norm.weight"], 1e-5) @ w["head.weight"].T

        handle = engine.claim()
        got, fed = [], 0
        for n_tok in (7, 2, 20, 1, 1, 19):
            got.append(engine.step([StepEntry(handle, toks[fed:fed + n_tok], list(range(n_tok)))]).cpu())
            fed += n_tok
        err = (torch.cat(got) - want).abs().max().item()
        assert err < 1e-4, err
    finally:
        FEED_FORWARDS.unregister("toy_routed")
        POSITION_ENCODINGS.unregister("toy_learned_offsets")
