"""Kernels timed alone, at the shapes of the Llama-3.1-8B layers by default.

    python -m torchllms_b200.kernels.microbench attention_decode
    python -m torchllms_b200.kernels.microbench attention_prefill --lengths 2048,8192 --impls mma,prefill
    python -m torchllms_b200.kernels.microbench gemm
    python -m torchllms_b200.kernels.microbench elementwise --tokens 2048
    python -m torchllms_b200.kernels.microbench peaks

Every case is timed with CUDA events after warm-up.  Memory-bound kernels run inside a CUDA
graph over several copies of their operands (more than the 126 MB of L2 together), so that a
launch does not find its inputs in L2 from the one before.  Figures go to standard output; the
summaries under ``profiles/`` quote them.
"""

from __future__ import annotations

import argparse
from typing import Callable, List

import torch

from . import get_ops

HEADS, KV_HEADS, HEAD_DIM, WIDTH, HIDDEN, VOCAB = 32, 8, 128, 4096, 14336, 128256


def _time(fn: Callable[[], None], reps: int) -> float:
    """Microseconds per call of ``fn``."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def _graphed(calls: List[Callable[[], None]]) -> Callable[[], None]:
    """One graph that makes every call once (they were warmed up before)."""
    for c in calls:
        c()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for c in calls:
            c()
    return g.replay


def attention_decode(args) -> None:
    """Decode attention (kernel and merge) for B requests of one context length."""
    ops = get_ops()
    copies = 8
    for spec in args.shapes.split(","):
        B, ctx = (int(x) for x in spec.split("x"))
        for page in (int(x) for x in args.pages.split(",")):
            torch.manual_seed(0)
            blocks = -(-ctx // page)
            table = torch.zeros(B, args.max_len // page, dtype=torch.int32)
            table[:, :blocks] = torch.randperm(B * blocks).view(B, blocks).int()
            table = table.cuda()
            caches = [(torch.randn(B * blocks, KV_HEADS, page, HEAD_DIM, device="cuda", dtype=torch.bfloat16),
                       torch.randn(B * blocks, KV_HEADS, page, HEAD_DIM, device="cuda", dtype=torch.bfloat16))
                      for _ in range(copies)]
            q = torch.randn(B, HEADS, HEAD_DIM, device="cuda", dtype=torch.bfloat16)
            q_start = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            kv_len = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
            out = torch.empty_like(q)

            def layer(i):
                k, v = caches[i]
                return lambda: ops.paged_attention(q, k, v, table, q_start, kv_len, n_seqs=B, max_q_len=1,
                                                   max_kv_len=args.max_len, scale=HEAD_DIM ** -0.5, window=None,
                                                   page_size=page, impl="decode", out=out)
            us = _time(_graphed([layer(i) for i in range(copies)]), 10) / copies
            nbytes = B * ctx * KV_HEADS * HEAD_DIM * 2 * 2
            print(f"attention_decode {B:3d} x {ctx:6d} page {page:3d}: {us:7.1f} us  {nbytes / us / 1e6:5.2f} TB/s")


def attention_prefill(args) -> None:
    """Causal attention of one whole prompt of L tokens."""
    ops = get_ops()
    page = 16
    for L in (int(x) for x in args.lengths.split(",")):
        torch.manual_seed(0)
        blocks = -(-L // page)
        table = torch.randperm(blocks).int().view(1, blocks).cuda()
        k = torch.randn(blocks, KV_HEADS, page, HEAD_DIM, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(blocks, KV_HEADS, page, HEAD_DIM, device="cuda", dtype=torch.bfloat16)
        q = torch.randn(L, HEADS, HEAD_DIM, device="cuda", dtype=torch.bfloat16)
        q_start = torch.tensor([0, L], dtype=torch.int32, device="cuda")
        kv_len = torch.tensor([L], dtype=torch.int32, device="cuda")
        out = torch.empty_like(q)
        flops = 4 * HEADS * HEAD_DIM * L * (L + 1) / 2
        for impl in args.impls.split(","):
            def call():
                ops.paged_attention(q, k, v, table, q_start, kv_len, n_seqs=1, max_q_len=L, max_kv_len=L,
                                    scale=HEAD_DIM ** -0.5, window=None, page_size=page, impl=impl, out=out)
            # ten launches in one graph: a short prompt's kernel takes less than the host needs to launch it
            us = _time(_graphed([call] * 10), 5) / 10
            ops.check_status()
            print(f"attention_prefill L {L:6d} {impl:8s}: {us:9.1f} us  {flops / us / 1e6:7.1f} TFLOP/s")


def gemm(args) -> None:
    """The projections of a decode step: x[M, K] . w[N, K]^T, the tcgen05 kernel beside torch.mm."""
    ops = get_ops()
    shapes = [("wo", WIDTH, WIDTH), ("w1;w3", 2 * HIDDEN, WIDTH), ("w2", WIDTH, HIDDEN),
              ("wq;wk;wv", (HEADS + 2 * KV_HEADS) * HEAD_DIM, WIDTH), ("head", VOCAB, WIDTH)]
    for M in (int(x) for x in args.rows.split(",")):
        for name, N, K in shapes:
            copies = max(2, int(300e6 // (N * K * 2)) + 1)
            ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            ours = _time(_graphed([(lambda w=w: ops.gemm_tcgen05(x, w, torch.float32)) for w in ws]), 5) / copies
            lib = _time(_graphed([(lambda w=w: torch.mm(x, w.t())) for w in ws]), 5) / copies
            ops.check_status()
            print(f"gemm M {M:3d} {name:9s} {N:6d} x {K:5d}: tcgen05 {ours:7.1f} us ({N * K * 2 / ours / 1e6:4.2f} TB/s)   "
                  f"torch.mm {lib:7.1f} us")


def elementwise(args) -> None:
    """Residual add + RMSNorm and SwiGLU over T tokens (bfloat16 activations, float32 stream)."""
    ops = get_ops()
    T, copies = args.tokens, 6
    hs = [torch.randn(T, WIDTH, device="cuda") for _ in range(copies)]
    ds = [torch.randn(T, WIDTH, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    w = torch.ones(WIDTH, device="cuda")
    us = _time(_graphed([(lambda i=i: ops.rmsnorm(hs[i], ds[i], w, 1e-5, torch.bfloat16)) for i in range(copies)]), 5) / copies
    print(f"rmsnorm T {T}: {us:7.1f} us  {T * WIDTH * 12 / us / 1e6:5.2f} TB/s")
    us = _time(_graphed([(lambda i=i: ops.rmsnorm(hs[i], ds[i], w, 1e-5, torch.bfloat16, deferred=True)) for i in range(copies)]), 5) / copies
    print(f"rmsnorm T {T}, scale deferred: {us:7.1f} us  {T * WIDTH * 12 / us / 1e6:5.2f} TB/s")
    # rotation of q and k and the write of k and v into pages, as a prompt portion of T tokens needs it
    row, page = (HEADS + 2 * KV_HEADS) * HEAD_DIM, 16
    qkvs = [torch.randn(T, row, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    table = torch.randn(T, HEAD_DIM // 2, 2, device="cuda")
    positions = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = torch.randperm(T, device="cuda").int()
    kp = torch.empty(-(-T // page), KV_HEADS, page, HEAD_DIM, device="cuda", dtype=torch.bfloat16)
    vp = torch.empty_like(kp)
    us = _time(_graphed([(lambda i=i: ops.rope_kv_write(qkvs[i], positions, table, n_heads=HEADS, n_kv_heads=KV_HEADS,
                                                        head_dim=HEAD_DIM, interleaved=True, k_pages=kp, v_pages=vp,
                                                        slot_mapping=slots, page_size=page)) for i in range(copies)]), 5) / copies
    print(f"rope + cache write T {T}: {us:7.1f} us  {T * row * 4 / us / 1e6:5.2f} TB/s")
    gus = [torch.randn(T, 2 * HIDDEN, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    us = _time(_graphed([(lambda i=i: ops.swiglu(gus[i])) for i in range(copies)]), 5) / copies
    print(f"swiglu  T {T}: {us:7.1f} us  {T * HIDDEN * 6 / us / 1e6:5.2f} TB/s")


def peaks(args) -> None:
    """What this GPU gives a plain copy and a library bfloat16 product: the denominators of a roofline."""
    n = 1 << 30
    src = torch.empty(n, dtype=torch.int32, device="cuda")
    dst = torch.empty_like(src)
    us = _time(lambda: dst.copy_(src), 10)
    print(f"copy of {4 * n / 1e9:.1f} GB: {us:9.1f} us  {2 * 4 * n / us / 1e6:5.2f} TB/s (read + write)")
    m = 8192
    a = torch.randn(m, m, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(m, m, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda: torch.mm(a, b), 10)
    print(f"library product {m}^3 bfloat16, ten in a row: {us:9.1f} us  {2 * m ** 3 / us / 1e6:7.1f} TFLOP/s")
    us = _time(lambda: torch.mm(a, b), 400)
    print(f"library product {m}^3 bfloat16, four hundred in a row: {us:9.1f} us  {2 * m ** 3 / us / 1e6:7.1f} TFLOP/s")


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="case", required=True)
    p = sub.add_parser("attention_decode")
    p.add_argument("--shapes", default="8x2048,64x2048,8x8192,32x8192,1x2048,1x8192", help="requests x context, comma separated")
    p.add_argument("--pages", default="16,64")
    p.add_argument("--max-len", type=int, default=8192)
    p.set_defaults(run=attention_decode)
    p = sub.add_parser("attention_prefill")
    p.add_argument("--lengths", default="2048,8192")
    p.add_argument("--impls", default="mma,prefill")
    p.set_defaults(run=attention_prefill)
    p = sub.add_parser("gemm")
    p.add_argument("--rows", default="8,64")
    p.set_defaults(run=gemm)
    p = sub.add_parser("peaks")
    p.set_defaults(run=peaks)
    p = sub.add_parser("elementwise")
    p.add_argument("--tokens", type=int, default=2048)
    p.set_defaults(run=elementwise)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the kernels need a CUDA device")
    args.run(args)


if __name__ == "__main__":
    main()
