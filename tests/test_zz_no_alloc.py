"""The attention entry point for callers that cannot allocate device memory.

Some users of this library are not allowed to call cudaMalloc while they run: an application that
gave the whole GPU to a memory pool of its own, a real-time loop that cannot afford the
device-wide synchronisation an allocation implies, a plug-in working inside another program's
stream.  For them ``tl_paged_attention_static_scratch`` keeps the split-KV partial results in an
8 MiB array that is part of the library itself.  This test calls it the way such a user would,
through the exported C symbol with raw device pointers, twice in a row on different inputs (the
array is shared and keeps the previous call's contents), and compares with the plain PyTorch twin
of the attention kernels and with the ordinary entry point, which is given a workspace.  It sits
last in the collection order on purpose.
"""

import ctypes

import pytest
import torch

from torch_ops import TorchOps

pytestmark = pytest.mark.gpu

TOO_SMALL = -40


def _step(seed, lens, H, KV, hd, P, dtype):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    blocks = [-(-n // P) for n in lens]
    n_pages = sum(blocks) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, max(blocks) + 1), -1, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for j in range(blocks[b]):
            table[b, j] = next(it)
    dev = lambda t: t.cuda()
    return dict(
        q=dev(torch.randn((B, H, hd), generator=g).to(dtype)),
        k_pages=dev(torch.randn((n_pages, KV, P, hd), generator=g).to(dtype)),
        v_pages=dev(torch.randn((n_pages, KV, P, hd), generator=g).to(dtype)),
        block_table=dev(table), q_start=dev(torch.arange(B + 1, dtype=torch.int32)),
        kv_len=dev(torch.tensor(lens, dtype=torch.int32)), n_seqs=B, max_q_len=1, max_kv_len=max(lens), page_size=P)


def _call_static(lib, a, out, scale, dtype_code):
    q = a["q"]
    T, H, hd = q.shape
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.tl_paged_attention_static_scratch(
        ptr(q), ptr(a["k_pages"]), ptr(a["v_pages"]), ptr(out), ptr(a["block_table"]), a["block_table"].stride(0),
        ptr(a["q_start"]), ptr(a["kv_len"]), dtype_code, T, a["n_seqs"], H, a["k_pages"].shape[1], hd, a["page_size"],
        a["max_q_len"], a["max_kv_len"], 0, ctypes.c_float(scale), 1,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 2e-5), (torch.bfloat16, 1, 2e-2)])
def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row(dtype, code, tol):
    from torchllms_b200.kernels import get_ops
    from torchllms_b200.kernels.build import load_library
    ops = get_ops()
    lib = load_library("attention")
    lib.tl_static_scratch_strerror.restype = ctypes.c_char_p
    H, KV, hd, P = 8, 2, 64, 16
    for seed, lens in ((1, [2000, 1700]), (2, [900, 2100, 640])):     # the second call finds the first one's leftovers
        a = _step(seed, lens, H, KV, hd, P, dtype)
        n_splits, floats = ctypes.c_int(0), ctypes.c_longlong(0)
        assert lib.tl_attention_plan(len(lens), len(lens), H, KV, hd, 1, max(lens), 1,
                                     ctypes.byref(n_splits), ctypes.byref(floats)) == 0
        assert n_splits.value > 1 and 0 < floats.value <= 2 * 1024 * 1024   # the scratch really is in use
        out = torch.full_like(a["q"], float("nan"))
        rc = _call_static(lib, a, out, hd ** -0.5, code)
        assert rc == 0, lib.tl_static_scratch_strerror(rc).decode()
        ordinary = ops.paged_attention(**a, scale=hd ** -0.5, window=None, impl="general")
        torch.cuda.synchronize()
        twin = TorchOps().paged_attention(**a, scale=hd ** -0.5, window=None)     # plain PyTorch, no kernel of ours
        torch.testing.assert_close(out.float(), twin.float(), atol=tol, rtol=tol)
        torch.testing.assert_close(out.float(), ordinary.float(), atol=tol, rtol=tol)


def test_static_scratch_refuses_what_does_not_fit():
    from torchllms_b200.kernels.build import load_library
    lib = load_library("attention")
    lib.tl_static_scratch_strerror.restype = ctypes.c_char_p
    # 290 requests x 16 heads of width 256, keys cut in two: 290 * 16 * 2 * 258 floats, more than the array holds
    a = _step(3, [300] * 290, 16, 1, 256, 16, torch.float32)
    n_splits, floats = ctypes.c_int(0), ctypes.c_longlong(0)
    lib.tl_attention_plan(290, 290, 16, 1, 256, 1, 300, 1, ctypes.byref(n_splits), ctypes.byref(floats))
    assert n_splits.value == 2 and floats.value > 2 * 1024 * 1024
    out = torch.full_like(a["q"], 7.0)
    rc = _call_static(lib, a, out, 0.1, 0)
    torch.cuda.synchronize()
    assert rc == TOO_SMALL and b"8 MiB" in lib.tl_static_scratch_strerror(rc)
    assert bool((out == 7.0).all())                                    # nothing was launched
