"""Each part of a layer alone on the GPU, built from its spec with numbers of its own, against the
plain implementation's function for that part."""

import math

import pytest
import torch

import plain_llama
from torchllms_b200.kernels.lazy import PendingProduct, RowScaled
from torchllms_b200.cache.manager import RunCacheView
from torchllms_b200.engine.step import StepContext
from torchllms_b200.parts import attention, block, ffn, norm, rope  # noqa: F401
from torchllms_b200.parts.base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, BuildEnv, Residual
from torchllms_b200.parts.spec import PartSpec, part

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def env_for(dim, dtype, max_positions=512):
    from torchllms_b200.kernels import get_ops
    return BuildEnv(dim=dim, dtype=dtype, device=torch.device("cuda"), max_positions=max_positions, ops=get_ops())


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)


def ctx_for(portions, starts, page_size, n_pages, device="cuda"):
    """A step context and block table for requests that bring ``portions[i]`` tokens starting at
    position ``starts[i]``; request i owns pages i*k .. in order (k pages each)."""
    B = len(portions)
    k = n_pages // B
    q_start = [0]
    for n in portions:
        q_start.append(q_start[-1] + n)
    pos = [s + j for s, n in zip(starts, portions) for j in range(n)]
    seq = [i for i, n in enumerate(portions) for _ in range(n)]
    table = torch.tensor([[i * k + b for b in range(k)] for i in range(B)], dtype=torch.int32)
    slots = [int(table[i, p // page_size]) * page_size + p % page_size for i, p in zip(seq, pos)]
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    kv = [s + n for s, n in zip(starts, portions)]
    ctx = StepContext(n_tokens=len(pos), n_seqs=B, n_want=0, max_q_len=max(portions), max_kv_len=max(kv), n_decode=0,
                      token_ids=t([0] * len(pos)), positions=t(pos), seq_of_token=t(seq), q_start=t(q_start),
                      kv_len=t(kv), state_slot=t(list(range(B))), fresh=t([int(s == 0) for s in starts]),
                      want_rows=t([]), q_lens=list(portions), kv_lens=kv, slots=list(range(B)))
    return ctx, table.to(device), t(slots)


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    env = env_for(200, dtype)
    n = NORMS.build(part("rmsnorm", dim=200, eps=3e-4), env)
    assert list(n.expected_tensors()) == ["weight"] and n.expected_tensors()["weight"].shape == (200,)
    w = 1 + 0.2 * torch.randn(200)
    n.load({"weight": w})
    h = torch.randn(9, 200, device="cuda") * 2
    delta = torch.randn(9, 200, device="cuda").to(dtype)
    res = Residual(h.clone(), delta)
    got = n.forward(res)
    assert res.delta is None and torch.equal(res.h, h + delta.float())
    want = plain_llama.rms_norm((h + delta.float()).cpu(), w, 3e-4)
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))
    assert got.dtype == dtype


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("scaling", [None, {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                           "high_freq_factor": 2.0, "original_max_position_embeddings": 32}])
def test_position_encoding_part(dtype, scaling):
    H, KV, hd, P = 5, 1, 48, 8
    env = env_for(64, dtype)
    pe = POSITION_ENCODINGS.build(part("rope", head_dim=hd, theta=1234.0, scaling=scaling, pairing="interleaved"), env)
    ctx, table, slots = ctx_for([7, 3], [0, 20], P, 8)
    qkv = torch.randn(10, (H + 2 * KV) * hd).to(dtype).cuda()
    k_pages = torch.zeros(8, KV, P, hd, dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    view = RunCacheView(k_pages, v_pages, table, slots, P, True, None)
    q = pe.encode_and_store(qkv, ctx, view, H, KV, hd)
    inv = plain_llama.rope_frequencies(hd, 1234.0, scaling)
    cos, sin = plain_llama.rope_angles(inv, ctx.positions.cpu())
    x = qkv.float().cpu().view(10, H + 2 * KV, hd)
    want_q = plain_llama.apply_rope(x[:, :H], cos, sin)
    want_k = plain_llama.apply_rope(x[:, H:H + KV], cos, sin)
    torch.testing.assert_close(q.float().cpu(), want_q, **tol(dtype))
    for t in range(10):
        page, slot = int(slots[t]) // P, int(slots[t]) % P
        torch.testing.assert_close(k_pages[page, :, slot].float().cpu(), want_k[t], **tol(dtype))
        assert torch.equal(v_pages[page, :, slot].cpu(), qkv[t].cpu().view(H + 2 * KV, hd)[H + KV:])


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    env = env_for(72, dtype)
    f = FEED_FORWARDS.build(part("swiglu", dim=72, hidden=200), env)
    w = {"w1.weight": torch.randn(200, 72) * 0.1, "w2.weight": torch.randn(72, 200) * 0.1, "w3.weight": torch.randn(200, 72) * 0.1}
    assert {k: v.shape for k, v in f.expected_tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    w = {k: v.to(dtype).float() for k, v in w.items()}
    f.load(w)
    x = torch.randn(11, 72).to(dtype)
    got = f.forward(x.cuda(), None)
    assert isinstance(got, PendingProduct)            # the down projection is left to the norm that follows
    got = got.take(env.ops)
    got = got.sum(0) if got.dim() == 3 else got
    want = plain_llama.swiglu_ffn(x.float(), w["w1.weight"], w["w2.weight"], w["w3.weight"])
    torch.testing.assert_close(got.float().cpu(), want, **tol(dtype))


def attention_weights(dim, H, KV, hd, dtype, scale=0.15):
    g = torch.Generator().manual_seed(5)
    w = {"wq.weight": torch.randn(H * hd, dim, generator=g) * scale, "wk.weight": torch.randn(KV * hd, dim, generator=g) * scale,
         "wv.weight": torch.randn(KV * hd, dim, generator=g) * scale, "wo.weight": torch.randn(dim, H * hd, generator=g) * scale}
    return {k: v.to(dtype).float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,P", [(6, 2, 16, 4), (3, 3, 32, 16)])
def test_attention_mixer_part_in_two_portions(dtype, H, KV, hd, P):
    dim, S, cut = 40, 45, 29
    env = env_for(dim, dtype)
    pos = part("rope", head_dim=hd, theta=500.0, scaling=None, pairing="interleaved")
    m = MIXERS.build(part("attention", dim=dim, n_heads=H, n_kv_heads=KV, head_dim=hd, scale=hd ** -0.5,
                          position=pos, window=None), env)
    need = m.cache_need()
    assert (need.kind, need.n_kv_heads, need.head_dim) == ("full", KV, hd) and m.state_need() is None
    w = attention_weights(dim, H, KV, hd, dtype)
    m.load(w)
    x = torch.randn(S, dim).to(dtype)
    n_pages = 16
    k_pages = torch.zeros(n_pages, KV, P, hd, dtype=dtype, device="cuda")
    v_pages = torch.zeros_like(k_pages)
    outs = []
    for start, n in ((0, cut), (cut, S - cut)):
        ctx, table, slots = ctx_for([n], [start], P, n_pages)
        view = RunCacheView(k_pages, v_pages, table, slots, P, True, None)
        outs.append(m.forward(x[start:start + n].cuda(), ctx, view).take(env.ops))    # (a pending output projection)
    got = torch.cat([(o.sum(0) if o.dim() == 3 else o).float() for o in outs]).cpu()
    cfg = {"n_heads": H, "n_kv_heads": KV, "head_dim": hd}
    cos, sin = plain_llama.rope_angles(plain_llama.rope_frequencies(hd, 500.0, None), torch.arange(S))
    stored = plain_llama._same if dtype == torch.float32 else plain_llama.to_bfloat16_and_back
    want = plain_llama.attention_layer(x.float(), w["wq.weight"], w["wk.weight"], w["wv.weight"], w["wo.weight"],
                                       cfg, cos, sin, stored)
    torch.testing.assert_close(got, want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_part(dtype):
    dim, H, KV, hd, hidden, P, S = 48, 4, 2, 16, 100, 8, 21
    env = env_for(dim, dtype)
    spec = part("prenorm",
                mixer=part("attention", dim=dim, n_heads=H, n_kv_heads=KV, head_dim=hd, scale=hd ** -0.5, window=None,
                           position=part("rope", head_dim=hd, theta=10000.0, scaling=None, pairing="interleaved")),
                feed_forward=part("swiglu", dim=dim, hidden=hidden),
                mixer_norm=part("rmsnorm", dim=dim, eps=1e-5), ffn_norm=part("rmsnorm", dim=dim, eps=1e-5),
                mixer_prefix="mix", ffn_prefix="ff", mixer_norm_prefix="n1", ffn_norm_prefix="n2")
    blk = BLOCKS.build(spec, env)
    names = blk.expected_tensors()
    assert set(names) == {"mix.wq.weight", "mix.wk.weight", "mix.wv.weight", "mix.wo.weight", "ff.w1.weight",
                          "ff.w2.weight", "ff.w3.weight", "n1.weight", "n2.weight"}
    g = torch.Generator().manual_seed(2)
    w = {k: ((1 + 0.1 * torch.randn(e.shape, generator=g)) if k.startswith("n") else torch.randn(e.shape, generator=g) * 0.15)
         for k, e in names.items()}
    w = {k: v.to(dtype).float() for k, v in w.items()}
    blk.load(w)
    x = torch.randn(S, dim)
    ctx, table, slots = ctx_for([S], [0], P, 4)
    k_pages = torch.zeros(4, KV, P, hd, dtype=dtype, device="cuda")
    view = RunCacheView(k_pages, torch.zeros_like(k_pages), table, slots, P, True, None)
    res = Residual(x.cuda().clone())
    blk.forward(res, ctx, view)
    delta = res.delta.take(env.ops).float()
    got = (res.h + (delta.sum(0) if delta.dim() == 3 else delta)).cpu()
    ren = {"mix.": "attention.", "ff.": "feed_forward.", "n1.": "attention_norm.", "n2.": "ffn_norm."}
    pw = {}
    for k, v in w.items():
        for a, b in ren.items():
            if k.startswith(a):
                pw["L." + b + k[len(a):]] = v
    cfg = {"n_heads": H, "n_kv_heads": KV, "head_dim": hd, "eps": 1e-5}
    cos, sin = plain_llama.rope_angles(plain_llama.rope_frequencies(hd, 10000.0, None), torch.arange(S))
    stored = plain_llama._same if dtype == torch.float32 else plain_llama.to_bfloat16_and_back
    want = plain_llama.block(x, pw, "L", cfg, cos, sin, stored)
    torch.testing.assert_close(got, want, **tol(dtype))


def test_norm_part_defers_its_scale_and_folds_a_pending_product_into_the_stream():
    """In bfloat16, for a reader that takes row-scaled input: the rows leave weighted, the scale beside
    them; a pending product is added to the stream by its own kernel when it has few rows, by product
    and norm kernel otherwise, with the same result."""
    dim, K = 256, 136
    env = env_for(dim, torch.bfloat16)
    n = NORMS.build(part("rmsnorm", dim=dim, eps=1e-5), env)
    w = 1 + 0.2 * torch.randn(dim)
    n.load({"weight": w})
    for rows in (9, 100):
        h = torch.randn(rows, dim, device="cuda") * 2
        x = torch.randn(rows, K, device="cuda").to(torch.bfloat16)
        wo = (torch.randn(dim, K, device="cuda") * 0.1).to(torch.bfloat16)
        product = (x.float() @ wo.float().t()).to(torch.bfloat16).float()
        res = Residual(h.clone(), PendingProduct(x, wo))
        got = n.forward(res, deferred_ok=True)
        assert isinstance(got, RowScaled) and res.delta is None and got.ssq.shape[1] == (8 if rows <= 64 else 1)
        assert (res.h - (h + product)).abs().max().item() <= 2.0 ** -7 * product.abs().max().item()
        want = plain_llama.rms_norm(res.h.cpu(), w, 1e-5)
        torch.testing.assert_close(got.resolve(torch.float32).cpu(), want, atol=3e-2, rtol=2e-2)
        plain_way = n.forward(Residual(h.clone(), PendingProduct(x, wo)))      # not deferred: the ordinary norm
        assert isinstance(plain_way, torch.Tensor)
        torch.testing.assert_close(plain_way.float().cpu(), want, atol=3e-2, rtol=2e-2)
    env32 = env_for(dim, torch.float32)
    n32 = NORMS.build(part("rmsnorm", dim=dim, eps=1e-5), env32)
    n32.load({"weight": w})
    out = n32.forward(Residual(torch.randn(4, dim, device="cuda")), deferred_ok=True)
    assert isinstance(out, torch.Tensor)                  # 32-bit mode keeps the reference's order


def test_unknown_kinds_are_named():
    env = env_for(8, torch.float32)
    with pytest.raises(KeyError, match="registered"):
        MIXERS.build(part("hyena"), env)
    with pytest.raises(Exception):
        MIXERS.build(part("attention", dim=8, n_heads=2, n_kv_heads=1, head_dim=24, scale=1.0,
                          position=part("rope", head_dim=24, theta=1.0)), env)       # head_dim no multiple of 16
