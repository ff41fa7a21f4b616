"""Plain PyTorch twins of the CUDA kernels, one function per kernel, same signatures.

They serve two purposes in the tests: each kernel is compared with its twin on
the GPU, and the engine's host-side logic (cache, step function, scheduler,
replay) is exercised on the CPU by building an engine over a :class:`TorchOps`.
Nothing in the package imports this file.
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from torchllms_b200.kernels.lazy import PendingProduct, RowScaled      # two value types, no kernels

MASK64 = (1 << 64) - 1


def mix64(z: int) -> int:
    z &= MASK64
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return z


def _mix64_np(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z ^ (z >> np.uint64(30))
        z = z * np.uint64(0xBF58476D1CE4E5B9)
        z = z ^ (z >> np.uint64(27))
        z = z * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    return z


def noise_row(key: int, vocab: int) -> np.ndarray:
    """-log(-log(u)) for every vocabulary index, as float32, from the 64-bit row key."""
    with np.errstate(over="ignore"):
        i = np.arange(1, vocab + 1, dtype=np.uint64)
        bits = _mix64_np(np.uint64(key & MASK64) + i * np.uint64(0x9E3779B97F4A7C15))
    u = ((bits >> np.uint64(41)).astype(np.float32) + np.float32(0.5)) * np.float32(2.0 ** -23)
    return (-np.log(-np.log(u))).astype(np.float32)


class TorchOps:
    name = "torch-twin"

    def prepare(self, dtype, sampling=True):
        pass

    def check_attention_sizes(self, n_heads, n_kv_heads, head_dim, dtype):
        assert n_heads % n_kv_heads == 0 and head_dim % 2 == 0

    def embed(self, token_ids, table):
        return table[token_ids.long()].float()

    def rmsnorm(self, h, delta, weight, eps, out_dtype, rows=None, deferred=False):
        if isinstance(delta, PendingProduct):
            delta = delta.take(self)
        if delta is not None and delta.dim() == 3:
            delta = delta.float().sum(0)
        x = h if delta is None else h + delta.float()
        if rows is None:
            if delta is not None:
                h.copy_(x)
        else:
            x = x[rows.long()]
        if deferred:
            assert rows is None
            return RowScaled((x * weight).to(out_dtype), x.pow(2).sum(-1, keepdim=True), x.shape[1], float(eps))
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight
        return y.to(out_dtype)

    fuse_residual = True      # tests switch it off to compare the two ways

    def can_fuse_residual(self, pending, h):
        return (self.fuse_residual and isinstance(pending, PendingProduct) and pending.x.dtype == torch.bfloat16
                and pending.x.shape[0] <= 64 and pending.w.shape[0] % 4 == 0 and pending.x.shape[1] % 8 == 0)

    def linear_residual_norm(self, pending, h, weight, eps, slab=128):
        """h += bf16(x @ w.T) (float32, in place); rows bf16(h * weight) and the sum of squares in parts
        of ``slab`` columns, as the kernel leaves them."""
        h += (pending.x.float() @ pending.w.float().t()).to(torch.bfloat16).float()
        N = h.shape[1]
        parts = [h[:, c:c + slab].pow(2).sum(-1) for c in range(0, N, slab)]
        return RowScaled((h * weight).to(torch.bfloat16), torch.stack(parts, 1), N, float(eps))

    def swiglu(self, gate_up, out_dtype=None):
        scale = None
        if isinstance(gate_up, RowScaled):
            scale, gate_up = gate_up.scale(), gate_up.x
        out_dtype = out_dtype or gate_up.dtype
        if gate_up.dim() == 3:
            gate_up = gate_up.float().sum(0)
        hidden = gate_up.shape[1] // 2
        g, u = gate_up[:, :hidden].float(), gate_up[:, hidden:].float()
        if scale is not None:
            g, u = g * scale[:, None], u * scale[:, None]
        return (g / (1 + torch.exp(-g)) * u).to(out_dtype)

    def linear_swiglu(self, x, w13, fused=None):
        if isinstance(x, RowScaled):
            # gate and up pass through the activation dtype unscaled, as between the product and its epilogue
            return self.swiglu(x.follow(self.linear(x.x, w13)), out_dtype=x.x.dtype)
        return self.swiglu(self.linear(x, w13), out_dtype=x.dtype)

    def linear(self, x, w, out_dtype=None, partials_ok=False):
        if isinstance(x, RowScaled):
            return x.follow(self.linear(x.x, w, out_dtype, partials_ok))
        out_dtype = out_dtype or x.dtype
        if x.dtype == torch.float32:
            return (x @ w.t()).to(out_dtype)
        return (x.float() @ w.float().t()).to(out_dtype)

    def gemm_simt(self, x, w, out_dtype):
        return (x.float() @ w.float().t()).to(out_dtype)

    def rope_kv_write(self, qkv, positions, table, *, n_heads, n_kv_heads, head_dim, interleaved,
                      k_pages, v_pages, slot_mapping, page_size, out_dtype=None):
        scale = None
        if isinstance(qkv, RowScaled):
            scale, qkv = qkv.scale(), qkv.x
        out_dtype = out_dtype or qkv.dtype
        if qkv.dim() == 3:
            qkv = qkv.float().sum(0)
        T = qkv.shape[0]
        x = qkv.float().view(T, n_heads + 2 * n_kv_heads, head_dim)
        if scale is not None:
            x = x * scale[:, None, None]
        cs = table[positions.long()]            # [T, hd/2, 2]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        rot = x[:, : n_heads + n_kv_heads]
        if interleaved:
            a, b = rot[..., 0::2], rot[..., 1::2]
        else:
            a, b = rot[..., : head_dim // 2], rot[..., head_dim // 2:]
        ya, yb = a * c - b * s, b * c + a * s
        out = torch.empty_like(rot)
        if interleaved:
            out[..., 0::2], out[..., 1::2] = ya, yb
        else:
            out[..., : head_dim // 2], out[..., head_dim // 2:] = ya, yb
        q = out[:, :n_heads].to(out_dtype).contiguous()
        if k_pages is not None:
            k = out[:, n_heads:].to(out_dtype)
            v = x[:, n_heads + n_kv_heads:].to(out_dtype)
            sm = slot_mapping.long()
            page, slot = sm // page_size, sm % page_size
            k_pages[page, :, slot] = k
            v_pages[page, :, slot] = v
        return q

    def paged_attention(self, q, k_pages, v_pages, block_table, q_start, kv_len, *, n_seqs, max_q_len,
                        max_kv_len, scale, window, page_size, allow_split=True, impl="auto", n_tokens=None, out=None):
        T, H, hd = q.shape
        KV = k_pages.shape[1]
        group = H // KV
        # the same contract as the kernels' front end: the step's bounds cover its requests and fit the table
        assert block_table.shape[1] * page_size >= max_kv_len, "block_table is too narrow for max_kv_len"
        assert int(kv_len[:n_seqs].max()) <= max_kv_len and n_seqs <= block_table.shape[0]
        out = torch.zeros_like(q) if out is None else out
        qs = q_start.tolist()
        kl = kv_len.tolist()
        for b in range(n_seqs):
            ql, L = qs[b + 1] - qs[b], kl[b]
            lo = 0
            if window:
                lo = max(0, (L - ql) - window + 1)
            pos = torch.arange(lo, L, device=q.device)
            pages = block_table[b].long()[pos // page_size]
            assert (pages >= 0).all(), "attention would read a page that was given back"
            k = k_pages[pages, :, pos % page_size].float()     # [n, KV, hd]
            v = v_pages[pages, :, pos % page_size].float()
            qq = q[qs[b]:qs[b + 1]].float()                    # [ql, H, hd]
            qpos = torch.arange(L - ql, L, device=q.device)
            hidden = pos[None, :] > qpos[:, None]
            if window:
                hidden = hidden | (pos[None, :] <= qpos[:, None] - window)
            for h in range(H):
                s = (qq[:, h] @ k[:, h // group].T) * scale
                s = s.masked_fill(hidden, float("-inf"))
                out[qs[b]:qs[b + 1], h] = (torch.softmax(s, -1) @ v[:, h // group]).to(q.dtype)
        return out

    def sample(self, logits, temperature=None, top_k=None, row_keys=None):
        n, vocab = logits.shape
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
        for r in range(n):
            row = logits[r].float().cpu()
            t = 0.0 if temperature is None else float(temperature[r])
            if not t > 0:
                out[r] = int(torch.argmax(row))
                continue
            score = row / np.float32(max(t, 1e-5))
            k = 0 if top_k is None else int(top_k[r])
            if 0 < k < vocab:
                pivot = torch.topk(row, k).values[-1]
                score = score.masked_fill(row < pivot, float("-inf"))
            key = int(row_keys[r]) & MASK64
            score = score + torch.from_numpy(noise_row(key, vocab))
            out[r] = int(torch.argmax(score))
        return out
