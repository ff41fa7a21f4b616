"""Each CUDA kernel alone against its plain PyTorch twin, at sizes other than the engine's."""

import math

import numpy as np
import pytest
import torch

from torch_ops import TorchOps, mix64, noise_row

pytestmark = pytest.mark.gpu

TWIN = TorchOps()
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from torchllms_b200.kernels import get_ops
    return get_ops()


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).cuda()


# ------------------------------------------------------------------------------ elementwise

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,dim,n", [(37, 24, 5), (1000, 96, 64), (50, 4100, 3), (300, 4096, 70), (9, 8, 2), (1003, 102, 9), (11, 7, 3)])
def test_embed(ops, dtype, vocab, dim, n):
    table = rand((vocab, dim), dtype, 1)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32).cuda()
    ids[0], ids[-1] = vocab - 1, 0
    out = ops.embed(ids, table)
    assert out.dtype == torch.float32
    assert torch.equal(out, TWIN.embed(ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,dim", [(1, 16), (7, 96), (33, 4096), (3, 5000), (2, 20000), (5, 102), (4, 7)])
@pytest.mark.parametrize("eps", [1e-5, 1e-2])
def test_rmsnorm_with_and_without_delta(ops, dtype, n, dim, eps):
    h = rand((n, dim), torch.float32, 2, 3.0)
    delta = rand((n, dim), dtype, 3)
    w = 1 + 0.1 * rand((dim,), torch.float32, 4)
    for d in (None, delta):
        h1, h2 = h.clone(), h.clone()
        got = ops.rmsnorm(h1, d, w, eps, out_dtype=dtype)
        want = TWIN.rmsnorm(h2, d, w, eps, out_dtype=dtype)
        assert got.dtype == dtype
        torch.testing.assert_close(got.float(), want.float(), atol=tol(dtype, 2e-5), rtol=tol(dtype, 1e-5, 1e-2))
        # the sum replaced the stream (exactly: it is one float32 addition per element)
        assert torch.equal(h1, h2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_rows_leaves_stream_alone(ops, dtype):
    h = rand((19, 200), torch.float32, 5)
    delta = rand((19, 200), dtype, 6)
    w = rand((200,), torch.float32, 7)
    rows = torch.tensor([18, 0, 7, 7], dtype=torch.int32).cuda()
    before = h.clone()
    got = ops.rmsnorm(h, delta, w, 1e-6, out_dtype=dtype, rows=rows)
    want = TWIN.rmsnorm(before.clone(), delta, w, 1e-6, out_dtype=dtype, rows=rows)
    assert torch.equal(h, before)
    torch.testing.assert_close(got.float(), want.float(), atol=tol(dtype, 2e-5), rtol=tol(dtype, 1e-5, 1e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,hidden", [(1, 8), (5, 192), (64, 1000), (3, 14336), (7, 166), (3, 5)])
def test_swiglu(ops, dtype, n, hidden):
    x = rand((n, 2 * hidden), dtype, 8, 3.0)
    got, want = ops.swiglu(x), TWIN.swiglu(x)
    torch.testing.assert_close(got.float(), want.float(), atol=tol(dtype, 1e-5), rtol=tol(dtype, 1e-5, 1e-2))


# ------------------------------------------------------------------------------------ gemm

@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (1, 1000, 96), (7, 65, 17), (64, 64, 16), (65, 129, 100),
                                   (200, 96, 4096), (3, 512, 14336)])
def test_gemm_simt_float32_is_true_32bit(ops, M, N, K):
    x, w = rand((M, K), torch.float32, 9), rand((N, K), torch.float32, 10)
    got = ops.linear(x, w)
    want = (x.double() @ w.double().t())
    err = (got.double() - want).abs().max().item()
    scale = want.abs().max().item() + 1e-6
    # float32 accumulation error grows like sqrt(K) * eps; a tf32 or bf16 product would be 1e-3 off
    assert err / scale < 2e-6 * math.sqrt(K) + 1e-6, (err, scale)


@pytest.mark.parametrize("M,N,K", [(1, 1000, 96), (7, 65, 17), (33, 130, 200)])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_gemm_simt_bfloat16_operands(ops, M, N, K, out_dtype):
    x, w = rand((M, K), torch.bfloat16, 11), rand((N, K), torch.bfloat16, 12)
    got = ops.gemm_simt(x, w, out_dtype)
    want = TWIN.gemm_simt(x, w, out_dtype)
    torch.testing.assert_close(got.float(), want.float(), atol=tol(out_dtype, 1e-4, 5e-2), rtol=tol(out_dtype, 1e-5, 1e-2))


@pytest.mark.parametrize("M,N,K", [(1, 1000, 96), (5, 128, 64), (300, 200, 264), (5, 166, 102), (70, 1003, 102), (3, 9, 7)])
def test_linear_bfloat16(ops, M, N, K):
    x, w = rand((M, K), torch.bfloat16, 13), rand((N, K), torch.bfloat16, 14)
    for out_dtype in DTYPES:
        got = ops.linear(x, w, out_dtype=out_dtype)
        assert got.dtype == out_dtype
        want = x.float() @ w.float().t()
        torch.testing.assert_close(got.float(), want, atol=tol(out_dtype, 1e-3, 8e-2), rtol=tol(out_dtype, 1e-4, 1e-2))


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(128, 64), (96, 96), (1000, 200), (6144, 4096), (4096, 14336), (300, 8)])
def test_gemm_tcgen05_few_rows(ops, M, N, K):
    """The tensor-core kernel for decode-sized products: partial sums over K splits add up to x @ w^T."""
    x, w = rand((M, K), torch.bfloat16, 40 + M), rand((N, K), torch.bfloat16, 41, 0.5)
    want = x.double() @ w.double().t()
    for out_dtype in DTYPES:
        got = ops.gemm_tcgen05(x, w, out_dtype)
        ops.check_status()
        if got.dim() == 3:
            assert got.dtype == torch.float32 and got.shape[1:] == (M, N)
            got = got.double().sum(0)
        else:
            assert got.dtype == out_dtype and got.shape == (M, N)
            got = got.double()
        scale = want.abs().max().item()
        bound = (2e-6 * math.sqrt(K) + 1e-6) if out_dtype == torch.float32 or K > 256 else 5e-3
        if out_dtype == torch.bfloat16 and got.dtype != torch.float64:
            bound = 5e-3
        err = (got - want).abs().max().item() / scale
        assert err < max(bound, 5e-3 if out_dtype == torch.bfloat16 else 0), (err, out_dtype)
    # the public entry: 2-D result whatever the splits, and partial sums on request
    y = ops.linear(x, w)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    torch.testing.assert_close(y.double(), want, atol=2e-2 * want.abs().max().item(), rtol=2e-2)
    parts = ops.linear(x, w, partials_ok=True)
    assert parts.dim() in (2, 3)


@pytest.mark.parametrize("M,hidden,K", [(1, 64, 64), (8, 192, 264), (16, 14336, 128), (17, 448, 1000), (33, 128, 4096), (40, 192, 264), (64, 1024, 520)])
def test_gated_product_is_product_then_swiglu(ops, M, hidden, K):
    """SwiGLU in the epilogue of the gate/up product: the same numbers as product + SwiGLU kernel,
    and both near the float32 formula.  Sizes that are no power of two, one to 64 rows, a K with a
    ragged last block, one slab and hundreds of them."""
    torch.manual_seed(M * 7 + hidden)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w13 = (torch.randn(2 * hidden, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    one = ops.linear_swiglu(x, w13, fused=True)
    two = ops.linear_swiglu(x, w13, fused=False)
    ops.check_status()
    gu = x.float() @ w13.float().t()
    g, u = gu[:, :hidden], gu[:, hidden:]
    want = g / (1 + torch.exp(-g)) * u
    assert one.dtype == torch.bfloat16 and one.shape == (M, hidden)
    torch.testing.assert_close(one.float(), want, atol=3e-2, rtol=3e-2)
    # two kernels: the product may be split over K (float32 partial sums, no rounding before the
    # activation), so equality is exact only where it is not
    lib = ops._lib("gemm_tcgen05")
    if lib.tl_gemm_tcgen05_splits(M, 2 * hidden, K) == 1:
        assert torch.equal(one, two)
    else:
        torch.testing.assert_close(one.float(), two.float(), atol=2e-2, rtol=2e-2)


def test_gemm_tcgen05_rows_do_not_depend_on_the_batch(ops):
    """A token's product is the same bits whatever else shares its bucket of rows (1-16, 17-32,
    33-64: the buckets split K differently, so across them results agree to float32 rounding)."""
    x, w = rand((64, 4096), torch.bfloat16, 50), rand((512, 4096), torch.bfloat16, 51, 0.3)
    sixteen = ops.gemm_tcgen05(x[:16].contiguous(), w, torch.float32)
    one = ops.gemm_tcgen05(x[5:6].contiguous(), w, torch.float32)
    assert torch.equal(sixteen[..., 5, :], one[..., 0, :])
    full = ops.gemm_tcgen05(x, w, torch.float32)
    some = ops.gemm_tcgen05(x[:40].contiguous(), w, torch.float32)
    assert torch.equal(full[..., :40, :], some)
    total = lambda t: t.sum(0) if t.dim() == 3 else t
    torch.testing.assert_close(total(full)[5], total(one)[0], atol=1e-4, rtol=1e-5)


# ------------------------------------------------- deferred normalisation and the product into the stream

from torchllms_b200.kernels.lazy import PendingProduct, RowScaled


def random_row_scale(T, parts, dim, seed):
    g = torch.Generator().manual_seed(seed)
    ssq = (torch.rand((T, parts), generator=g) * dim / parts * 4 + 0.01).cuda()
    return ssq, dim, 1e-5


@pytest.mark.parametrize("n,dim", [(1, 16), (7, 96), (33, 4096), (5, 102), (300, 128)])
def test_rmsnorm_deferred_leaves_weighted_rows_and_their_sums_of_squares(ops, n, dim):
    h = rand((n, dim), torch.float32, 2, 3.0)
    w = 1 + 0.1 * rand((dim,), torch.float32, 4)
    parts = rand((3, n, dim), torch.float32, 5)
    for delta in (None, rand((n, dim), torch.bfloat16, 3), parts):
        h1, h2 = h.clone(), h.clone()
        got = ops.rmsnorm(h1, delta, w, 1e-5, out_dtype=torch.bfloat16, deferred=True)
        want = TWIN.rmsnorm(h2, delta, w, 1e-5, out_dtype=torch.bfloat16, deferred=True)
        assert isinstance(got, RowScaled) and got.x.dtype == torch.bfloat16 and got.ssq.shape == (n, 1) and got.dim == dim
        torch.testing.assert_close(h1, h2, atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(got.x.float(), want.x.float(), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(got.ssq, want.ssq, atol=1e-3, rtol=1e-5)
        # resolved, it is the ordinary norm
        plain = TWIN.rmsnorm(h.clone(), delta, w, 1e-5, out_dtype=torch.float32)
        torch.testing.assert_close(got.resolve(torch.float32), plain, atol=3e-2, rtol=1e-2)


@pytest.mark.parametrize("M", [1, 8, 16, 17, 40, 64])
@pytest.mark.parametrize("N,K", [(128, 64), (132, 72), (4096, 4096), (4096, 14336), (300, 8), (1000, 200), (131, 520)])
def test_product_added_to_the_stream_in_its_own_kernel(ops, M, N, K):
    """h += bf16(x @ w^T), bf16(h * weight) and the parts of sum(h^2) from one kernel, in which the K
    splits of a column slab add up through the shared memory of their cluster: against the twin,
    against product + norm kernel, three times in a row, and bit for bit whatever the timing."""
    x, w = rand((M, K), torch.bfloat16, 60 + M), rand((N, K), torch.bfloat16, 61, K ** -0.5)
    h0 = rand((M, N), torch.float32, 62, 2.0)
    nw = 1 + 0.1 * rand((N,), torch.float32, 63)
    pending = PendingProduct(x, w)
    assert ops.can_fuse_residual(pending, h0) == (M <= ops.FUSE_MAX_ROWS)      # (the kernel takes up to 64 rows; the policy stops earlier)
    first = None
    for _ in range(3):
        h1, h2, h3 = h0.clone(), h0.clone(), h0.clone()
        got = ops.linear_residual_norm(pending, h1, nw, 1e-5)
        ops.check_status()
        want = TWIN.linear_residual_norm(pending, h2, nw, 1e-5)
        two = ops.rmsnorm(h3, ops.linear(x, w), nw, 1e-5, out_dtype=torch.bfloat16, deferred=True)   # product, then norm kernel
        assert got.x.shape == (M, N) and got.ssq.shape[0] == M and got.ssq.shape[1] == 4 * (-(-N // 128)) and got.dim == N
        # the product is rounded to bfloat16 on its way into the stream: where the float32 sums of two
        # orders fall on different sides of a rounding step, h differs by that step
        step = 2.0 ** -7 * (x.float() @ w.float().t()).abs().max().item()
        assert (h1 - h2).abs().max().item() <= step and (h1 - h3).abs().max().item() <= step
        assert ((h1 - h2).abs() > 1e-6).float().mean().item() < 0.02
        torch.testing.assert_close(got.x.float(), (h1 * nw).to(torch.bfloat16).float(), atol=0, rtol=0)
        torch.testing.assert_close(got.ssq.sum(-1), h1.pow(2).sum(-1), atol=1e-3, rtol=1e-5)
        torch.testing.assert_close(got.scale(), want.scale(), atol=1e-6, rtol=1e-4)
        torch.testing.assert_close(got.scale(), two.scale(), atol=1e-6, rtol=1e-4)
        if first is None:
            first = (h1.clone(), got.x.clone(), got.ssq.clone())
        else:
            assert torch.equal(h1, first[0]) and torch.equal(got.x, first[1]) and torch.equal(got.ssq, first[2])
    assert not ops.can_fuse_residual(PendingProduct(rand((65, K), torch.bfloat16, 1), w), torch.zeros(65, N, device="cuda"))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,P,interleaved", [(4, 2, 16, 16, True), (5, 5, 48, 4, False), (32, 8, 128, 16, True)])
@pytest.mark.parametrize("parts", [1, 32, 5])
def test_rope_applies_a_deferred_row_scale(ops, dtype, H, KV, hd, P, interleaved, parts):
    T, n_pages, max_pos = 19, 8, 100
    row = (H + 2 * KV) * hd
    pos = torch.randint(0, max_pos, (T,), dtype=torch.int32).cuda()
    ang = torch.arange(max_pos).float()[:, None] * (1.0 / 100 ** (torch.arange(hd // 2).float() / (hd // 2)))[None, :]
    table = torch.stack([ang.cos(), ang.sin()], -1).contiguous().cuda()
    slots = torch.randperm(n_pages * P)[:T].to(torch.int32).cuda()
    ssq, dim, eps = random_row_scale(T, parts, 256, 7)
    kw = dict(n_heads=H, n_kv_heads=KV, head_dim=hd, interleaved=interleaved, slot_mapping=slots, page_size=P, out_dtype=dtype)
    for qkv in (rand((T, row), dtype, 15), rand((4, T, row), torch.float32, 16)):
        pages = [torch.zeros((n_pages, KV, P, hd), dtype=dtype).cuda() for _ in range(4)]
        q1 = ops.rope_kv_write(RowScaled(qkv, ssq, dim, eps), pos, table, k_pages=pages[0], v_pages=pages[1], **kw)
        q2 = TWIN.rope_kv_write(RowScaled(qkv, ssq, dim, eps), pos, table, k_pages=pages[2], v_pages=pages[3], **kw)
        a = tol(dtype, 2e-5, 2e-2)
        torch.testing.assert_close(q1.float(), q2.float(), atol=a, rtol=a)
        torch.testing.assert_close(pages[0].float(), pages[2].float(), atol=a, rtol=a)
        torch.testing.assert_close(pages[1].float(), pages[3].float(), atol=a, rtol=a)
        unscaled = ops.rope_kv_write(qkv, pos, table, k_pages=None, v_pages=None, **kw)
        assert not torch.allclose(unscaled.float(), q1.float(), atol=a)


@pytest.mark.parametrize("M,hidden,K", [(1, 64, 64), (8, 192, 264), (16, 14336, 128), (33, 128, 4096), (64, 1024, 520), (9, 83, 40), (200, 256, 128)])
@pytest.mark.parametrize("parts", [1, 32])
def test_swiglu_applies_a_deferred_row_scale(ops, M, hidden, K, parts):
    """Gate and up of rows whose normalisation was deferred: the scale goes on before the activation,
    in the product's epilogue where there is one, in the SwiGLU kernel else; both against the twin."""
    torch.manual_seed(M + hidden)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w13 = (torch.randn(2 * hidden, K, device="cuda") * K ** -0.5).to(torch.bfloat16)
    ssq, dim, eps = random_row_scale(M, parts, K, 9)
    rs = RowScaled(x, ssq, dim, eps)
    want = TWIN.linear_swiglu(rs, w13)
    got = ops.linear_swiglu(rs, w13)
    ops.check_status()
    assert got.dtype == torch.bfloat16 and got.shape == (M, hidden)
    torch.testing.assert_close(got.float(), want.float(), atol=3e-2, rtol=3e-2)
    can_fuse = M <= 64 and hidden % 64 == 0 and K % 8 == 0
    if can_fuse:
        one, two = ops.linear_swiglu(rs, w13, fused=True), ops.linear_swiglu(rs, w13, fused=False)
        torch.testing.assert_close(one.float(), two.float(), atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(one.float(), want.float(), atol=3e-2, rtol=3e-2)
    # and it is the activation of the scaled product, not the scaled activation
    s = rs.scale()[:, None]
    gu = (x.float() @ w13.float().t()) * s
    ref = gu[:, :hidden] / (1 + torch.exp(-gu[:, :hidden])) * gu[:, hidden:]
    torch.testing.assert_close(got.float(), ref, atol=5e-2, rtol=5e-2)


# ------------------------------------------------------------------------------------ rope

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,P", [(4, 2, 16, 16), (3, 1, 32, 8), (5, 5, 48, 4), (32, 8, 128, 16)])
@pytest.mark.parametrize("interleaved", [True, False])
def test_rope_kv_write(ops, dtype, H, KV, hd, P, interleaved):
    T, n_pages, max_pos = 37, 12, 300
    qkv = rand((T, (H + 2 * KV) * hd), dtype, 15)
    pos = torch.randint(0, max_pos, (T,), dtype=torch.int32).cuda()
    ang = torch.arange(max_pos).float()[:, None] * (1.0 / 100 ** (torch.arange(hd // 2).float() / (hd // 2)))[None, :]
    table = torch.stack([ang.cos(), ang.sin()], -1).contiguous().cuda()
    slots = torch.randperm(n_pages * P)[:T].to(torch.int32).cuda()
    pages = [torch.full((n_pages, KV, P, hd), 7.0, dtype=dtype).cuda() for _ in range(4)]
    kw = dict(n_heads=H, n_kv_heads=KV, head_dim=hd, interleaved=interleaved, slot_mapping=slots, page_size=P)
    q1 = ops.rope_kv_write(qkv, pos, table, k_pages=pages[0], v_pages=pages[1], **kw)
    q2 = TWIN.rope_kv_write(qkv, pos, table, k_pages=pages[2], v_pages=pages[3], **kw)
    a = tol(dtype, 1e-5, 2e-2)
    torch.testing.assert_close(q1.float(), q2.float(), atol=a, rtol=a)
    torch.testing.assert_close(pages[0].float(), pages[2].float(), atol=a, rtol=a)
    assert torch.equal(pages[1], pages[3])          # values are copied bit for bit
    assert (pages[0] == 7.0).any()                   # untouched slots stay untouched
    # a run that reads another run's cache writes nothing
    q3 = ops.rope_kv_write(qkv, pos, table, k_pages=None, v_pages=None, **kw)
    assert torch.equal(q1, q3)


# ------------------------------------------------------------------------------- attention

def build_paged(seq_lens, q_lens, H, KV, hd, P, dtype, seed, n_extra_pages=3, peak=None):
    """Random queries and a shuffled page pool holding random keys/values for each request."""
    g = torch.Generator().manual_seed(seed)
    B = len(seq_lens)
    blocks = [-(-L // P) for L in seq_lens]
    n_pages = sum(blocks) + n_extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_blocks = max(blocks) + 2
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    k_pages = torch.randn((n_pages, KV, P, hd), generator=g)
    v_pages = torch.randn((n_pages, KV, P, hd), generator=g)
    it = iter(perm)
    for b in range(B):
        for j in range(blocks[b]):
            table[b, j] = next(it)
    T = sum(q_lens)
    q = torch.randn((T, H, hd), generator=g)
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    if peak is not None:
        # make one far key dominate: the query of (request b, head h) becomes a multiple of that key
        b, key_pos, boost = peak
        page, slot = table[b, key_pos // P].item(), key_pos % P
        for h in range(H):
            q[q_start[b]:q_start[b + 1], h] = boost * k_pages[page, h // (H // KV), slot]
    dev = lambda t: t.cuda()
    return dict(q=dev(q.to(dtype)), k_pages=dev(k_pages.to(dtype)), v_pages=dev(v_pages.to(dtype)),
                block_table=dev(table), q_start=dev(q_start),
                kv_len=dev(torch.tensor(seq_lens, dtype=torch.int32)), n_seqs=B,
                max_q_len=max(q_lens), max_kv_len=max(seq_lens), page_size=P)


ATTN_CASES = [
    # seq_lens, q_lens, H, KV, hd, P, window
    ([5], [5], 4, 2, 16, 16, None),                       # one short prompt
    ([33, 1, 64, 7], [33, 1, 64, 7], 4, 2, 16, 16, None), # whole prompts, ragged
    ([40, 100, 17], [1, 1, 1], 3, 1, 32, 8, None),        # decode, group of 3
    ([90, 41, 64, 130], [24, 1, 2, 1], 3, 1, 32, 8, None),  # portions beside decoded tokens
    ([70, 9], [70, 3], 6, 2, 48, 4, None),                # head_dim 48, page 4
    ([300, 257], [300, 1], 8, 2, 64, 16, None),
    ([129, 50], [2, 50], 32, 8, 128, 16, None),           # the 8B head layout
    ([77], [5], 20, 1, 16, 16, None),                     # 20 query heads on one kv head (> 16 rows)
    ([100, 60], [100, 1], 2, 2, 256, 32, None),           # head_dim 256, no grouping
    ([200, 90, 33], [200, 1, 5], 4, 2, 32, 8, 17),        # sliding window over page edges
    ([64, 65], [64, 1], 4, 4, 16, 16, 16),                # window exactly one page
    ([1000, 300, 5], [1, 1, 1], 32, 8, 128, 16, None),    # decoding in the 8B head layout
    ([500, 77], [3, 2], 8, 2, 64, 16, None),              # portions so short that a request's rows fit one tile
    ([150], [150], 10, 2, 32, 8, None),                   # group of 5: 3 tokens to a 16-row tile, one row idle
    ([90, 20], [90, 1], 16, 1, 64, 16, None),             # group of 16
    ([700, 650], [1, 1], 4, 2, 32, 16, 100),              # decoding behind a window
    ([2100], [2100], 8, 8, 128, 16, None),                # a long prompt, many key tiles
    ([333, 64, 1, 65, 2000], [1, 1, 1, 1, 1], 8, 2, 128, 4, None),    # decoding, pages of 4
    ([333, 64, 1, 65, 2000], [1, 1, 1, 1, 1], 6, 2, 64, 8, None),     # decoding, group of 3, pages of 8
    ([900, 130], [2, 1], 16, 2, 64, 32, 77),              # two tokens of a group of 8 behind a window, pages of 32
    ([300, 5], [1, 1], 4, 4, 128, 128, None),             # pages larger than a tile
    ([1500, 1499, 3], [1, 1, 1], 32, 8, 128, 16, 512),    # the 8B layout decoding behind a window
    ([700, 45], [3, 4], 32, 8, 128, 16, None),            # 16 rows to a tile (four tokens of a group of four), head_dim 128
    ([400, 33, 130], [1, 1, 1], 16, 1, 128, 16, None),    # decoding with a group of 16, head_dim 128
    ([260, 19], [2, 1], 12, 2, 64, 8, 50),                # group of 6: two tokens make 12 rows, behind a window
    ([3000, 700], [400, 700], 8, 2, 128, 16, None),       # a portion late in a long context beside a whole prompt
    ([1000], [1000], 4, 2, 64, 32, 300),                  # a window that spans several key tiles
    ([600, 130], [600, 129], 4, 4, 128, 256, None),       # pages larger than a key tile of any kernel
    ([1200], [1200], 8, 2, 128, 16, 200),                 # head_dim 128 behind a window that starts inside a key tile
    ([700, 300, 1025], [700, 300, 1025], 8, 2, 128, 16, None),   # ragged whole prompts: a last query block of one row
    ([2500, 520], [257, 384], 4, 1, 64, 64, 1000),        # portions late in their contexts, windowed, pages of 64
    ([1500 + 7 * i for i in range(64)], [1] * 64, 8, 2, 128, 16, None),   # decoding over more keys and values than L2 holds (their copies are marked to leave it first)
]


IMPLS = [(torch.float32, "general"), (torch.bfloat16, "general"), (torch.bfloat16, "mma"), (torch.bfloat16, "decode"),
         (torch.bfloat16, "prefill"), (torch.bfloat16, "prefill2")]


def mma_takes(hd):
    return hd in (16, 32, 64, 128)


def prefill_takes(hd, P):
    return hd in (64, 128) and P & (P - 1) == 0


def decode_takes(q_lens, H, KV, hd, P):
    group = H // KV
    return hd in (64, 128) and P & (P - 1) == 0 and max(q_lens) <= 16 // min(group, 16)


@pytest.mark.parametrize("dtype,impl", IMPLS)
@pytest.mark.parametrize("case", ATTN_CASES, ids=[str(i) for i in range(len(ATTN_CASES))])
def test_paged_attention_matches_twin(ops, dtype, impl, case):
    seq_lens, q_lens, H, KV, hd, P, window = case
    if impl == "mma" and not mma_takes(hd):
        pytest.skip("the tensor-core kernel does not take this head size")
    if impl == "decode" and not decode_takes(q_lens, H, KV, hd, P):
        pytest.skip("the decode kernel does not take this step")
    if impl in ("prefill", "prefill2") and not prefill_takes(hd, P):
        pytest.skip("the tcgen05 prefill kernel does not take this head size or page size")
    a = build_paged(seq_lens, q_lens, H, KV, hd, P, dtype, seed=len(seq_lens) * 100 + hd)
    scale = hd ** -0.5
    got = ops.paged_attention(**a, scale=scale, window=window, impl=impl)
    want = TWIN.paged_attention(**a, scale=scale, window=window)
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(got.float(), want.float(), atol=t, rtol=t)


@pytest.mark.parametrize("dtype,impl", IMPLS)
@pytest.mark.parametrize("B,L", [(1, 2000), (2, 777), (3, 4100)])
def test_decode_attention_split_over_keys(ops, dtype, impl, B, L):
    """Few long requests: the key range is split over CTAs and merged; same answer as unsplit."""
    lens = [L - 13 * i for i in range(B)]
    a = build_paged(lens, [1] * B, 8, 2, 64, 16, dtype, seed=L)
    split = ops.paged_attention(**a, scale=0.125, window=None, allow_split=True, impl=impl)
    whole = ops.paged_attention(**a, scale=0.125, window=None, allow_split=False, impl=impl)
    want = TWIN.paged_attention(**a, scale=0.125, window=None)
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(split.float(), want.float(), atol=t, rtol=t)
    torch.testing.assert_close(whole.float(), want.float(), atol=t, rtol=t)


@pytest.mark.parametrize("n_splits", [2, 3, 6, 8, 12])
@pytest.mark.parametrize("case", [
    ([2000, 1987, 300], [1, 1, 1], 8, 2, 64, 16, None),
    ([1000, 130, 5, 64], [1, 1, 1, 1], 32, 8, 128, 16, None),     # short requests leave some splits without keys
    ([700, 45], [3, 4], 32, 8, 128, 16, None),                    # 16 rows to a tile
    ([1500, 1499, 3], [1, 1, 1], 32, 8, 128, 16, 512),            # behind a window
    ([900, 130], [2, 1], 16, 2, 64, 32, 77),                      # a window narrower than the splits
], ids=["hd64", "8b", "rows16", "window", "narrow"])
def test_decode_attention_with_a_given_number_of_splits(ops, case, n_splits):
    """However many CTAs share a request's keys, the merged result is what one CTA per request
    gives, also where some splits see no key at all."""
    seq_lens, q_lens, H, KV, hd, P, window = case
    a = build_paged(seq_lens, q_lens, H, KV, hd, P, torch.bfloat16, seed=n_splits)
    scale = hd ** -0.5
    got = ops.paged_attention(**a, scale=scale, window=window, allow_split=n_splits, impl="decode")
    whole = ops.paged_attention(**a, scale=scale, window=window, allow_split=False, impl="decode")
    want = TWIN.paged_attention(**a, scale=scale, window=window)
    ops.check_status()
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.float(), whole.float(), atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype,impl", IMPLS)
@pytest.mark.parametrize("key_pos", [0, 15, 16, 511, 640])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype, impl, key_pos):
    """Random scores hide a dropped key; here one key takes nearly all the weight, so the output
    must equal that key's value."""
    L, H, KV, hd, P = 700, 4, 2, (64 if impl in ("decode", "prefill", "prefill2") else 32), 16
    a = build_paged([L, 40], [1, 1], H, KV, hd, P, dtype, seed=key_pos, peak=(0, key_pos, 10.0))
    got = ops.paged_attention(**a, scale=hd ** -0.5, window=None, impl=impl).float()
    page, slot = a["block_table"][0, key_pos // P].item(), key_pos % P
    for h in range(H):
        v = a["v_pages"][page, h // (H // KV), slot].float()
        assert (got[0, h] - v).abs().max().item() < 0.05, (h, (got[0, h] - v).abs().max().item())
    want = TWIN.paged_attention(**a, scale=hd ** -0.5, window=None).float()
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(got, want, atol=t, rtol=t)


@pytest.mark.parametrize("dtype,impl", [(torch.float32, "general"), (torch.bfloat16, "general"), (torch.bfloat16, "decode")])
@pytest.mark.parametrize("key_pos", [5, 12345, 32767])
def test_decoding_finds_one_key_among_tens_of_thousands(ops, dtype, impl, key_pos):
    """Decoding at a context of 32,768 in the 8-billion-parameter head layout: block tables of
    thousands of pages, the keys of a request split over as many CTAs as the plan gives at that
    length, and one key, early, in the middle or the very last, that takes nearly all the weight."""
    L, H, KV, hd, P = 32768, 32, 8, 128, 16
    a = build_paged([L, 20000], [1, 1], H, KV, hd, P, dtype, seed=key_pos, peak=(0, key_pos, 4.0))
    got = ops.paged_attention(**a, scale=hd ** -0.5, window=None, impl=impl).float()
    ops.check_status()
    page, slot = a["block_table"][0, key_pos // P].item(), key_pos % P
    for h in range(H):
        v = a["v_pages"][page, h // (H // KV), slot].float()
        assert (got[0, h] - v).abs().max().item() < 0.05, (h, (got[0, h] - v).abs().max().item())
    want = TWIN.paged_attention(**a, scale=hd ** -0.5, window=None).float()
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(got, want, atol=t, rtol=t)


@pytest.mark.parametrize("dtype,impl", IMPLS)
@pytest.mark.parametrize("key_pos", [0, 127, 128, 300, 511, 640])
def test_a_long_portion_finds_one_far_key(ops, dtype, impl, key_pos):
    """The same for a portion of hundreds of rows late in a longer context (several query tiles and
    key tiles, two query tiles to a CTA in the tcgen05 kernel, pages in shuffled order): every row
    that can see the key must return its value, every row before it must not."""
    if impl == "decode":
        pytest.skip("the decode kernel takes no long portions")
    L, Q, H, KV, hd, P = 700, 600, 4, 2, (64 if impl in ("prefill", "prefill2") else 32), 16
    a = build_paged([L, 40], [Q, 1], H, KV, hd, P, dtype, seed=key_pos + 1, peak=(0, key_pos, 10.0))
    got = ops.paged_attention(**a, scale=hd ** -0.5, window=None, impl=impl).float()
    page, slot = a["block_table"][0, key_pos // P].item(), key_pos % P
    first_row = L - Q                                     # position of the portion's first token
    for h in range(H):
        v = a["v_pages"][page, h // (H // KV), slot].float()
        err = (got[:Q, h] - v).abs().amax(dim=1)          # per row
        sees = torch.arange(first_row, L, device=err.device) >= key_pos
        assert (err[sees] < 0.06).all(), (h, int(torch.nonzero(err * sees >= 0.06)[0]))
        if (~sees).any():
            assert (err[~sees] > 0.06).all()
    want = TWIN.paged_attention(**a, scale=hd ** -0.5, window=None).float()
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(got, want, atol=t, rtol=t)


@pytest.mark.parametrize("dtype,impl", IMPLS)
def test_window_edge_is_exact(ops, dtype, impl):
    """The key just outside the window gets a huge score: if the edge were off by one it would
    take over the output."""
    L, H, KV, hd, P, w = 100, 2, 1, (64 if impl in ("decode", "prefill", "prefill2") else 16), 8, 24
    for edge_inside in (False, True):
        key_pos = (L - 1) - w + (1 if edge_inside else 0)   # last query sits at L - 1
        a = build_paged([L], [1], H, KV, hd, P, dtype, seed=3, peak=(0, key_pos, 12.0))
        got = ops.paged_attention(**a, scale=hd ** -0.5, window=w, impl=impl).float()
        page, slot = a["block_table"][0, key_pos // P].item(), key_pos % P
        v = a["v_pages"][page, 0, slot].float()
        close = (got[0, 0] - v).abs().max().item() < 0.05
        assert close == edge_inside
        want = TWIN.paged_attention(**a, scale=hd ** -0.5, window=w).float()
        torch.testing.assert_close(got, want, atol=tol(dtype, 2e-5, 2e-2), rtol=tol(dtype, 2e-5, 2e-2))


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_prefill_attention_on_random_shapes(ops, seed):
    """Both tcgen05 prefill kernels on shapes nobody picked: heads and groups, page sizes from 4 to 256, up to
    four requests whose portions start anywhere in their contexts, windows of any length."""
    import random
    rng = random.Random(seed)
    for _ in range(40):
        hd = rng.choice([64, 128])
        KV = rng.choice([1, 2, 4, 8])
        H = KV * rng.choice([1, 2, 4, 8])
        P = rng.choice([4, 8, 16, 32, 64, 128, 256])
        q_lens = [rng.choice([rng.randint(96, 300), rng.randint(1, 700), rng.randint(200, 1100)]) for _ in range(rng.randint(1, 4))]
        seq_lens = [q + rng.choice([0, 0, rng.randint(1, 1500)]) for q in q_lens]
        window = rng.choice([None, None, rng.randint(1, 900)])
        a = build_paged(seq_lens, q_lens, H, KV, hd, P, torch.bfloat16, seed=rng.randrange(1 << 30))
        want = TWIN.paged_attention(**a, scale=hd ** -0.5, window=window).float()
        for impl in ("prefill", "prefill2"):
            got = ops.paged_attention(**a, scale=hd ** -0.5, window=window, impl=impl).float()
            ops.check_status()
            torch.testing.assert_close(got, want, atol=2e-2, rtol=2e-2, msg=lambda m: f"{impl} {seq_lens} {q_lens} H{H} KV{KV} hd{hd} P{P} w{window}: {m}")


def test_attention_refuses_sizes_it_cannot_do(ops):
    from torchllms_b200.kernels.native import KernelError
    with pytest.raises(KernelError):
        ops.check_attention_sizes(4, 2, 24, torch.float32)     # head_dim no multiple of 16
    with pytest.raises(KernelError):
        ops.check_attention_sizes(4, 3, 32, torch.float32)     # heads no multiple of kv heads
    with pytest.raises(KernelError):
        ops.check_attention_sizes(4, 2, 512, torch.bfloat16)   # too wide
    with pytest.raises(KernelError):
        ops.embed(torch.zeros(3, dtype=torch.int32), torch.zeros(4, 4))  # CPU tensors


def test_a_wait_that_nothing_satisfies_gives_up_and_reports(ops):
    """The tensor-core and TMA kernels wait on mbarriers with a time limit and report through a
    status word instead of hanging.  A kernel with one such wait, which nothing will ever
    satisfy, shows the mechanism: it returns after the limit, the status says so, and the device
    goes on working."""
    from torchllms_b200.kernels.native import KernelError
    ops.check_status()                                   # clean before
    waited = ops.wait_selftest(limit_ms=2.0)
    assert 2.0 <= waited < 50.0, waited
    with pytest.raises(KernelError, match="gave up waiting"):
        ops.check_status()
    ops.check_status()                                   # the word was cleared
    x = torch.randn(8, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    got = ops.linear(x, w)                               # the context is alive and the kernels still run
    got = got.sum(0) if got.dim() == 3 else got
    torch.testing.assert_close(got.float(), (x.float() @ w.float().t()), atol=0.5, rtol=2e-2)
    ops.check_status()


# -------------------------------------------------------------------------------- sampling

def test_greedy_is_first_argmax(ops):
    logits = rand((9, 1000), torch.float32, 20)
    logits[3, 17] = logits[3, 900] = 50.0    # a tie: the lower index wins
    logits[4, 999] = 60.0
    got = ops.sample(logits)
    assert got.tolist() == torch.argmax(logits, -1).tolist()
    assert got[3].item() == 17 and got[4].item() == 999


@pytest.mark.parametrize("vocab", [50, 1000, 128256])
def test_sampling_matches_twin(ops, vocab):
    n = 6
    logits = rand((n, vocab), torch.float32, 21, 2.0)
    temp = torch.tensor([0.0, 0.7, 1.0, 1.3, 0.8, 1e-7], dtype=torch.float32).cuda()
    top_k = torch.tensor([0, 0, 5, vocab + 3, 1, 0], dtype=torch.int32).cuda()
    keys = torch.tensor([mix64(i + 77) - (1 << 63) for i in range(n)], dtype=torch.int64).cuda()
    got = ops.sample(logits, temp, top_k, keys).tolist()
    want = TWIN.sample(logits, temp, top_k, keys).tolist()
    # log differs by an ulp between the GPU and numpy: accept the GPU's choice if its twin score is the best within 1e-4
    for r in range(n):
        if got[r] != want[r]:
            t = max(float(temp[r]), 1e-5)
            score = logits[r].cpu().numpy() / np.float32(t) + noise_row(int(keys[r]) & ((1 << 64) - 1), vocab)
            assert abs(score[got[r]] - score[want[r]]) < 1e-4 * max(1.0, abs(score[want[r]]))
    assert got[0] == int(torch.argmax(logits[0]))       # temperature 0 is greedy
    assert got[4] == int(torch.argmax(logits[4]))       # top-1 is greedy
    assert got[5] == int(torch.argmax(logits[5]))       # a vanishing temperature is clamped, hence greedy


@pytest.mark.parametrize("vocab", [8193, 50000, 128256])
def test_sampling_without_top_k_over_many_ctas(ops, vocab):
    """Large vocabularies without a rank filter take the two-stage kernels: same answers."""
    n = 5
    logits = rand((n, vocab), torch.float32, 31, 2.0)
    logits[1, 4095] = logits[1, 4096] = logits[1, vocab - 1] = 40.0        # a tie across chunk borders
    assert ops.sample(logits).tolist() == torch.argmax(logits, -1).tolist()
    assert ops.sample(logits)[1].item() == 4095
    temp = torch.tensor([0.0, 0.9, 1.0, 0.5, 2.0], dtype=torch.float32).cuda()
    keys = torch.tensor([mix64(i + 5) - (1 << 63) for i in range(n)], dtype=torch.int64).cuda()
    got = ops.sample(logits, temp, None, keys).tolist()
    want = TWIN.sample(logits, temp, None, keys).tolist()
    for r in range(n):
        if got[r] != want[r]:
            t = max(float(temp[r]), 1e-5)
            score = logits[r].cpu().numpy() / np.float32(t) + noise_row(int(keys[r]) & ((1 << 64) - 1), vocab)
            assert abs(score[got[r]] - score[want[r]]) < 1e-4 * max(1.0, abs(score[want[r]]))
    # and the single-CTA kernel, asked through a top_k that filters nothing, agrees
    top_k = torch.zeros(n, dtype=torch.int32).cuda()
    assert ops.sample(logits, temp, top_k, keys).tolist() == got


def test_sampling_follows_the_softmax(ops):
    """Frequencies over many keys approach softmax(logits / T), and top-k never leaves its set."""
    vocab, n = 12, 20000
    base = torch.tensor([2.0, 1.0, 0.5, 0.0, -0.5, -1.0, 1.5, -3.0, 0.2, 0.1, -0.1, 0.7])
    logits = base[None, :].repeat(n, 1).cuda()
    temp = torch.full((n,), 0.8, dtype=torch.float32).cuda()
    keys = torch.tensor([mix64(1234567 * i + 1) - (1 << 63) for i in range(n)], dtype=torch.int64).cuda()
    got = ops.sample(logits, temp, None, keys).cpu().numpy()
    freq = np.bincount(got, minlength=vocab) / n
    p = torch.softmax(base / 0.8, -1).numpy()
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() / n) + 2e-3
    top_k = torch.full((n,), 3, dtype=torch.int32).cuda()
    got3 = ops.sample(logits, temp, top_k, keys).cpu().numpy()
    assert set(np.unique(got3)) <= {0, 1, 6}
    p3 = torch.softmax(base[[0, 1, 6]] / 0.8, -1).numpy()
    f3 = np.array([(got3 == i).mean() for i in (0, 1, 6)])
    assert np.abs(f3 - p3).max() < 0.02
