"""Pages that a window has passed are given back and belong to somebody else: no attention kernel
may look them up.  Here the block tables hold no page (-1) for every block that lies wholly before
the first key the step can see, and every page that no table names is filled with NaN, so that a
kernel that fetched one (even to multiply it by a probability of zero) would show it.

(The file sorts late, so that a run that stops at the first failure has seen the older tests.)"""

import pytest
import torch

from test_kernels_gpu import IMPLS, TWIN, build_paged, decode_takes, mma_takes, prefill_takes, tol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from torchllms_b200.kernels import get_ops
    return get_ops()


CASES = [
    # seq_lens, q_lens, H, KV, hd, P, window
    ([1000, 40], [300, 40], 4, 2, 64, 16, 200),          # a long portion late in a context: key tiles start before the window does
    ([1500, 700], [1, 1], 8, 2, 128, 16, 512),           # decoding behind a window
    ([900, 130], [2, 1], 16, 2, 64, 32, 77),             # two tokens, pages of 32
    ([2000], [700], 8, 8, 128, 16, 130),                 # several query tiles, each with a window start of its own
    ([640, 300], [128, 5], 4, 2, 64, 128, 100),          # pages as large as a key tile
]


@pytest.mark.parametrize("dtype,impl", IMPLS)
@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_pages_behind_a_window_are_never_looked_up(ops, dtype, impl, case):
    seq_lens, q_lens, H, KV, hd, P, window = case
    if impl == "mma" and not mma_takes(hd):
        pytest.skip("the tensor-core kernel does not take this head size")
    if impl == "decode" and not decode_takes(q_lens, H, KV, hd, P):
        pytest.skip("the decode kernel does not take this step")
    if impl == "prefill" and not (prefill_takes(hd, P) and max(q_lens) >= 96):
        pytest.skip("the tcgen05 prefill kernel does not take this step")
    a = build_paged(seq_lens, q_lens, H, KV, hd, P, dtype, seed=7)
    table = a["block_table"].clone()
    gone = 0
    for b, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        first_seen = max(0, (L - ql) - window + 1)       # the first key of the step's first query
        for j in range(first_seen // P):                 # blocks that end before it
            table[b, j] = -1
            gone += 1
    assert gone > 0
    named = set(table[table >= 0].tolist())
    for page in range(a["k_pages"].shape[0]):
        if page not in named:
            a["k_pages"][page] = float("nan")
            a["v_pages"][page] = float("nan")
    a["block_table"] = table
    scale = hd ** -0.5
    got = ops.paged_attention(**a, scale=scale, window=window, impl=impl)
    ops.check_status()
    assert torch.isfinite(got.float()).all()
    want = TWIN.paged_attention(**a, scale=scale, window=window)      # (asserts that it reads no page that is gone)
    t = tol(dtype, 2e-5, 2e-2)
    torch.testing.assert_close(got.float(), want.float(), atol=t, rtol=t)
