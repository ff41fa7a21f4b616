"""Choosing next tokens for a batch of requests: greedy, temperature, optional top-k.

Reference: ``sample`` (torchllms/inference/utils.py:36-48): temperature 0 is argmax; otherwise
logits / max(T, 1e-5), optional top-k cut, softmax, and ``argmax(probs / Exp(1))``
(:18-33).  The reference draws its noise from PyTorch's global generator, so a request's sample
depends on what else is in the batch.  Here the noise of a row is a pure function of
(seed, request, index of the generated token), computed inside the kernel, so a request samples
the same tokens alone or batched, whole or in portions, before or after a pre-emption.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def mix64(z: int) -> int:
    """The 64-bit finaliser the sampling kernel uses (same constants, same shifts)."""
    z &= MASK64
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & MASK64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return z


def row_key(seed: int, request: int, token_index: int) -> int:
    """Key of the noise for the ``token_index``-th generated token of ``request``."""
    return mix64((seed & MASK64) ^ mix64((request & MASK64) ^ mix64((token_index + GOLDEN) & MASK64)))


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: Optional[int] = None
    seed: int = 0


class PendingTokens:
    """Sampled tokens on their way to the host."""

    __slots__ = ("host", "done")

    def __init__(self, host: torch.Tensor, done):
        self.host, self.done = host, done


class Sampler:
    def __init__(self, ops, device):
        self.ops = ops
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], requests: Sequence[int],
               token_indices: Sequence[int]) -> List[int]:
        """One token per row of ``logits`` ``[n, vocab]`` (float32, on the device)."""
        return self.finish(self.launch(logits, params, requests, token_indices))

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], requests: Sequence[int],
               token_indices: Sequence[int]) -> torch.Tensor:
        """Start sampling and return the tokens as a device tensor without waiting for them:
        the caller may do host work before :meth:`finish` reads them back."""
        n = logits.shape[0]
        assert n == len(params) == len(requests) == len(token_indices)
        if all(not p.temperature > 0 for p in params):
            return self.ops.sample(logits)
        packed = np.zeros((n, 4), dtype=np.int32)  # temperature bits | top_k | key low | key high
        packed[:, 0] = np.asarray([p.temperature for p in params], dtype=np.float32).view(np.int32)
        packed[:, 1] = [int(p.top_k or 0) for p in params]
        keys = np.asarray([row_key(p.seed, r, t) for p, r, t in zip(params, requests, token_indices)], dtype=np.uint64)
        packed[:, 2:4] = keys.view(np.int32).reshape(n, 2)
        host = torch.from_numpy(packed)
        if self.device.type == "cuda":
            host = host.pin_memory()        # a copy from pageable memory would wait for the device
        dev = host.to(self.device, non_blocking=True)
        temperature = dev[:, 0].contiguous().view(torch.float32)
        # without a rank filter in the batch the kernel library may spread a row over many CTAs
        top_k = dev[:, 1].contiguous() if any((p.top_k or 0) > 0 for p in params) else None
        row_keys = dev[:, 2:4].contiguous().view(torch.int64).reshape(n)
        return self.ops.sample(logits, temperature, top_k, row_keys)

    def read_back(self, tokens: torch.Tensor) -> "PendingTokens":
        """Start copying the tokens of :meth:`launch` to the host.  Work queued on the device after
        this call does not delay :meth:`finish`, which waits for this copy alone."""
        if tokens.device.type != "cuda":
            return PendingTokens(tokens, None)
        host = torch.empty(tokens.shape, dtype=tokens.dtype, pin_memory=True)
        host.copy_(tokens, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return PendingTokens(host, done)

    def finish(self, tokens) -> List[int]:
        """The tokens of :meth:`launch` (or of :meth:`read_back`) on the host; this waits for them."""
        if isinstance(tokens, PendingTokens):
            if tokens.done is not None:
                tokens.done.synchronize()
            return self._checked(tokens.host.tolist())
        return self._checked(tokens.tolist())

    def _checked(self, tokens: List[int]) -> List[int]:
        # the device has finished everything up to the read-back: a kernel that gave up a wait has said so by now
        check = getattr(self.ops, "check_status", None)
        if check is not None:
            check()
        return tokens
