"""ctypes front end of the CUDA kernels: argument checks, output allocation, launches.

Every method checks dtype, device, contiguity and the sizes its kernel supports
and raises :class:`KernelError` with the reason; a size a kernel cannot handle
is refused, never computed wrongly.  Launches go to PyTorch's current stream,
so they order with PyTorch's own work and can be captured into CUDA graphs.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import functools
from typing import Dict, Optional, Tuple

import torch

from .build import ALL_LIBRARIES, build_libraries, load_library
from .lazy import PendingProduct, RowScaled

_DT = {torch.float32: 0, torch.bfloat16: 1}

_STATUS = {
    -1: "unsupported dtype",
    -2: "unsupported size",
    -3: "misaligned pointer",
    -4: "needs more shared memory or scratch than available",
}


class KernelError(RuntimeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  Asked for at every launch, so by the short way where this
    torch has it (the Stream object costs some 15 us to build, more than the launch itself)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: {_STATUS.get(rc, 'error ' + str(rc))}")
    raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no GPU'})")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_contig(t: torch.Tensor, name: str, dtype=None) -> None:
    _need(t.is_cuda, f"{name} must live on the GPU (there is no CPU implementation)")
    _need(t.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _need(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")


def _scale_args(rs: Optional[RowScaled], n_rows: int):
    """The four trailing arguments by which a kernel learns of rows whose normalisation was deferred."""
    if rs is None:
        return ctypes.c_void_p(0), 0, ctypes.c_float(0.0), ctypes.c_float(0.0)
    ssq = rs.ssq
    _need(ssq.is_cuda and ssq.dtype == torch.float32 and ssq.dim() == 2 and ssq.is_contiguous() and ssq.shape[0] >= n_rows,
          "row scale: ssq must be a contiguous float32 [rows, parts] tensor on the GPU")
    return _ptr(ssq), int(ssq.shape[1]), ctypes.c_float(1.0 / rs.dim), ctypes.c_float(rs.eps)


def _timed(fn):
    """While a profile is being taken, bracket the call with CUDA events."""
    name = fn.__name__

    @functools.wraps(fn)
    def wrapper(self, *args, **kwargs):
        prof = self._profile
        if prof is None:
            return fn(self, *args, **kwargs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        depth, self._profile_depth = self._profile_depth, self._profile_depth + 1
        a.record()
        try:
            out = fn(self, *args, **kwargs)
        finally:
            self._profile_depth = depth
        b.record()
        prof.append((name, a, b, depth))      # depth: a call made inside another is taken off the outer one's time
        return out
    return wrapper


class NativeOps:
    """The kernels as methods.  Libraries are compiled and loaded on first use."""

    PREFILL_MIN_Q = 96      # portions at least this long go to the tcgen05 prefill attention kernel
    FUSE_MAX_ROWS = 16      # steps of at most this many tokens let a product add itself to the residual stream and
                            # prepare the norm that follows in its own kernel; with more rows product + norm
                            # kernel are as fast or faster (measured: 16 rows equal, 32 and 64 rows 2 to 7 % slower)

    name = "native-sm100a"

    def __init__(self):
        if not torch.cuda.is_available():
            raise KernelError(
                "torchllms_b200 runs on a CUDA GPU (sm_100a) only: torch.cuda.is_available() is False "
                "and there is no CPU implementation")
        self.launches = 0          # kernels of this library launched so far (a bench counts with it)
        self._workspace: Dict[Tuple[int, str], torch.Tensor] = {}
        self._retired: list = []
        self.use_tcgen05 = True
        # SwiGLU in the epilogue of the gate/up product (TORCHLLMS_B200_NO_GATED=1 keeps the two kernels, for comparisons)
        self.use_gated = os.environ.get("TORCHLLMS_B200_NO_GATED", "") not in ("1", "true")
        # error word of kernels with bounded waits: pinned host memory the device writes to directly
        self._status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._mm_out_dtype: Optional[bool] = None
        self._profile = None
        self._profile_depth = 0
        # TORCHLLMS_B200_DEBUG=1: the libraries are built with -DTL_DEBUG (see kernels/build.py); kernels
        # range-check the indices they are given and report through a word that check_status() reads
        self.debug = os.environ.get("TORCHLLMS_B200_DEBUG", "") not in ("", "0")
        # the tcgen05 prefill attention multiplies probabilities as one bfloat16 (1: the faster kernel) or as
        # bfloat16 value + bfloat16 remainder (2: a third slower, half the rounding error)
        self.prefill_probability_parts = int(os.environ.get("TORCHLLMS_B200_PREFILL_PARTS", "1"))
        self.use_fused_residual = os.environ.get("TORCHLLMS_B200_NO_FUSED_RESIDUAL", "") not in ("1", "true")

    def graph_capturable(self, dtype: torch.dtype) -> bool:
        """Whether this library's launches for ``dtype`` may be recorded into a CUDA graph (not in
        debug mode: the limits its checks compare with are copied in from the host before launches)."""
        return not self.debug

    def _debug_limit(self, lib_name: str, which: int, value: int) -> None:
        """Debug builds: tell a library how many pages (0) or rows (1) the tensors of the next launch have."""
        if self.debug:
            _check(self._lib(lib_name).tl_debug_set_limit(which, ctypes.c_longlong(int(value)), _stream()), "debug limit")

    # ------------------------------------------------------------ libraries
    def prepare(self, dtype: torch.dtype, sampling: bool = True) -> None:
        """Compile, side by side, what a model of this dtype will call."""
        names = ["elementwise", "rope", "attention", "gemm_simt"]
        if dtype == torch.bfloat16:
            names += ["attention_mma", "attention_decode", "gemm_tcgen05"]
        if sampling:
            names.append("sampling")
        build_libraries(names)

    def _lib(self, name: str):
        return load_library(name)

    @contextlib.contextmanager
    def profile(self):
        """Time every call made inside the block; yields a dict name -> [calls, milliseconds]
        that is filled when the block ends (the stream is synchronised then)."""
        result: Dict[str, list] = {}
        self._profile = []
        try:
            yield result
        finally:
            records, self._profile = self._profile, None
            torch.cuda.synchronize()
            inner: Dict[int, float] = {}            # time of finished calls by depth, not yet taken off their caller
            for name, a, b, depth in records:       # (a call made inside another finishes, and is listed, first)
                ms = a.elapsed_time(b)
                entry = result.setdefault(name, [0, 0.0])
                entry[0] += 1
                entry[1] += ms - inner.pop(depth + 1, 0.0)
                inner[depth] = inner.get(depth, 0.0) + ms

    # ------------------------------------------------------------- checks
    def check_attention_sizes(self, n_heads: int, n_kv_heads: int, head_dim: int, dtype: torch.dtype) -> None:
        _need(dtype in _DT, f"attention supports float32 and bfloat16, not {dtype}")
        _need(n_heads > 0 and n_kv_heads > 0 and n_heads % n_kv_heads == 0,
              f"n_heads ({n_heads}) must be a positive multiple of n_kv_heads ({n_kv_heads})")
        _need(head_dim % 16 == 0 and 16 <= head_dim <= 256,
              f"head_dim must be a multiple of 16 between 16 and 256, got {head_dim}")

    # ------------------------------------------------------------ elementwise
    @_timed
    def embed(self, token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        _cuda_contig(token_ids, "token_ids", torch.int32)
        _cuda_contig(table, "embedding table")
        _need(table.dtype in _DT and table.dim() == 2, "embedding table must be a float32/bfloat16 matrix")
        n, (vocab, dim) = token_ids.numel(), table.shape
        out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
        rc = self._lib("elementwise").tl_embed(_ptr(token_ids), _ptr(table), _DT[table.dtype], _ptr(out),
                                              n, dim, vocab, _stream())
        _check(rc, "embed")
        self.launches += 1
        return out

    @_timed
    def rmsnorm(self, h: torch.Tensor, delta, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None, deferred: bool = False):
        """``delta`` may be a tensor, float32 partial sums ``[splits, T, dim]``, or a
        :class:`PendingProduct` (taken here the ordinary way).  ``deferred``: return the rows
        weighted but not normalised, as a :class:`RowScaled` (not with ``rows``)."""
        if isinstance(delta, PendingProduct):
            delta = delta.take(self)
        _cuda_contig(h, "residual stream", torch.float32)
        _cuda_contig(weight, "norm weight", torch.float32)
        _need(h.dim() == 2 and weight.numel() == h.shape[1], "norm weight must match the stream's width")
        _need(out_dtype in _DT, f"norm output dtype {out_dtype} unsupported")
        _need(not (deferred and rows is not None), "a deferred norm leaves whole streams, not gathered rows")
        dim = h.shape[1]
        _need(dim * 4 <= 200 * 1024, f"rmsnorm keeps a row in shared memory: width {dim} exceeds 51200")
        splits, plane = 1, 0
        if delta is not None:
            _cuda_contig(delta, "delta")
            _need(delta.dtype in _DT, "delta must be float32 or bfloat16")
            if delta.dim() == 3:          # partial sums of a split-K product, added up by the kernel
                _need(delta.shape[1:] == h.shape and delta.dtype == torch.float32,
                      "partial sums must be float32 [splits, tokens, width]")
                splits, plane = delta.shape[0], delta.stride(0)
            else:
                _need(delta.shape == h.shape, "delta must have the stream's shape")
        if rows is not None:
            _cuda_contig(rows, "rows", torch.int32)
        n_out = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n_out, dim), dtype=out_dtype, device=h.device)
        ssq = torch.empty((n_out, 1), dtype=torch.float32, device=h.device) if deferred else None
        write_back = 1 if (delta is not None and rows is None) else 0
        self._debug_limit("elementwise", 1, h.shape[0])
        rc = self._lib("elementwise").tl_rmsnorm(
            _ptr(h), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, splits, ctypes.c_longlong(plane),
            _ptr(weight), _ptr(out), _DT[out_dtype], _ptr(rows), n_out, dim, ctypes.c_float(eps), write_back,
            _ptr(ssq), _stream())
        _check(rc, "rmsnorm")
        self.launches += 1
        return RowScaled(out, ssq, dim, float(eps)) if deferred else out

    def can_fuse_residual(self, pending, h: torch.Tensor) -> bool:
        """Whether :meth:`linear_residual_norm` takes this pending product for this stream."""
        if not (self.use_fused_residual and self.use_tcgen05 and isinstance(pending, PendingProduct)):
            return False
        x, w = pending.x, pending.w
        if not (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2):
            return False
        M, K = x.shape
        N = w.shape[0]
        if not (h.shape == (M, N) and x.is_contiguous() and w.is_contiguous() and x.data_ptr() % 16 == 0
                and w.data_ptr() % 16 == 0 and M <= self.FUSE_MAX_ROWS):
            return False
        return self._lib("gemm_tcgen05").tl_gemm_tcgen05_residual_supports(M, N, K) == 1

    @_timed
    def linear_residual_norm(self, pending: PendingProduct, h: torch.Tensor, weight: torch.Tensor, eps: float) -> RowScaled:
        """``h += bf16(x @ w.T)`` in place (float32; the product rounded as one that passes through
        memory is) and the rows ``bf16(h * weight)`` with the parts of their sums of squares: one kernel in which the K splits of a column slab are one cluster of
        CTAs that add up through each other's shared memory."""
        x, w = pending.x, pending.w
        _cuda_contig(x, "linear input", torch.bfloat16)
        _cuda_contig(w, "linear weight", torch.bfloat16)
        _cuda_contig(h, "residual stream", torch.float32)
        _cuda_contig(weight, "norm weight", torch.float32)
        M, K = x.shape
        N = w.shape[0]
        _need(w.shape[1] == K and h.shape == (M, N) and weight.numel() == N, "linear_residual_norm: shapes disagree")
        lib = self._lib("gemm_tcgen05")
        _need(lib.tl_gemm_tcgen05_residual_supports(M, N, K) == 1,
              "the fused form takes bfloat16, at most 64 rows and K % 8 == 0")
        xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        ssq = torch.empty((M, lib.tl_gemm_tcgen05_residual_parts(N)), dtype=torch.float32, device=x.device)
        rc = lib.tl_gemm_tcgen05_residual(_ptr(x), _ptr(w), _ptr(h), _ptr(weight), _ptr(xw), _ptr(ssq), M, N, K,
                                          ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_residual")
        self.launches += 1
        return RowScaled(xw, ssq, N, float(eps))

    @_timed
    def swiglu(self, gate_up, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``gate_up`` is ``[tokens, 2 * hidden]``, or float32 partial sums ``[splits, tokens, 2 * hidden]``
        (then ``out_dtype`` says what to produce), or a :class:`RowScaled` of either (the scale is
        applied to gate and up before the activation)."""
        rs = gate_up if isinstance(gate_up, RowScaled) else None
        if rs is not None:
            gate_up = rs.x
        _cuda_contig(gate_up, "gate_up")
        _need(gate_up.dim() in (2, 3) and gate_up.shape[-1] % 2 == 0 and gate_up.dtype in _DT,
              "swiglu input must be [tokens, 2 * hidden] in float32/bfloat16")
        splits = gate_up.shape[0] if gate_up.dim() == 3 else 1
        _need(splits == 1 or gate_up.dtype == torch.float32, "partial sums must be float32")
        out_dtype = out_dtype or gate_up.dtype
        _need(out_dtype in _DT and (out_dtype == gate_up.dtype or gate_up.dtype == torch.float32),
              "swiglu cannot widen bfloat16 input")
        n, hidden = gate_up.shape[-2], gate_up.shape[-1] // 2
        out = torch.empty((n, hidden), dtype=out_dtype, device=gate_up.device)
        rc = self._lib("elementwise").tl_swiglu(_ptr(gate_up), _DT[gate_up.dtype], splits, _ptr(out), _DT[out_dtype],
                                               n, hidden, *_scale_args(rs, n), _stream())
        _check(rc, "swiglu")
        self.launches += 1
        return out

    # ------------------------------------------------------------------ linear
    @_timed
    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               partials_ok: bool = False) -> torch.Tensor:
        """``x [M, K] @ w[N, K]^T``.  float32 runs on the CUDA cores (true 32-bit).  bfloat16 with
        at most 64 rows (decode steps) runs on the tcgen05 kernel that streams the weight once;
        more rows use the library product, as the reference's ``nn.Linear`` does.

        With ``partials_ok`` the result may be float32 partial sums ``[splits, M, N]`` of a
        split-K product, for callers that hand it to a kernel which adds them up (residual +
        norm, rope, swiglu).  A :class:`RowScaled` input gives a :class:`RowScaled` result: the
        product is taken of the rows as they are and the scale follows it."""
        if isinstance(x, RowScaled):
            return x.follow(self.linear(x.x, w, out_dtype, partials_ok))
        _cuda_contig(x, "linear input")
        _cuda_contig(w, "linear weight")
        _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], "linear: inner sizes differ")
        _need(x.dtype == w.dtype and x.dtype in _DT, f"linear: dtypes {x.dtype} / {w.dtype} unsupported")
        out_dtype = out_dtype or x.dtype
        M, K = x.shape
        N = w.shape[0]
        if x.dtype == torch.float32:
            _need(out_dtype == torch.float32, "a float32 product has float32 output")
            return self.gemm_simt(x, w, torch.float32)
        if self.use_tcgen05 and M <= 64 and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            parts = self.gemm_tcgen05(x, w, out_dtype)
            if parts.dim() == 2 or partials_ok:
                return parts
            return parts.sum(0).to(out_dtype)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, w.t())
        _need(out_dtype == torch.float32, f"linear: output dtype {out_dtype} unsupported")
        if self._mm_out_dtype is None:
            try:
                torch.mm(x[:1], w[:8].t(), out_dtype=torch.float32)
                self._mm_out_dtype = True
            except (TypeError, RuntimeError):
                self._mm_out_dtype = False
        if self._mm_out_dtype and K % 8 == 0:              # (rows the library can address 16 bytes at a time)
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return self.gemm_simt(x, w, torch.float32)

    def linear_swiglu(self, x: torch.Tensor, w13: torch.Tensor, fused: Optional[bool] = None) -> torch.Tensor:
        """``silu(x @ w13[:H]^T) * (x @ w13[H:]^T)`` for a stacked gate/up weight ``[2 H, K]``, in
        ``x``'s dtype.  Decode-sized bfloat16 inputs whose product needs no K split run as one
        kernel (the activation in the product's epilogue); everything else as product + SwiGLU
        kernel, with the same numbers.  ``fused`` forces the choice (tests).  ``x`` may be a
        :class:`RowScaled`: gate and up are scaled before the activation."""
        rs = x if isinstance(x, RowScaled) else None
        if rs is not None:
            x = rs.x
        _cuda_contig(x, "linear input")
        _cuda_contig(w13, "linear weight")
        _need(x.dim() == 2 and w13.dim() == 2 and x.shape[1] == w13.shape[1] and w13.shape[0] % 2 == 0,
              "linear_swiglu: x [M, K] against w13 [2 H, K]")
        M, K = x.shape
        hidden = w13.shape[0] // 2
        can = (x.dtype == torch.bfloat16 and w13.dtype == torch.bfloat16 and self.use_tcgen05 and M <= 64 and hidden % 64 == 0
               and K % 8 == 0 and K >= 8 and x.data_ptr() % 16 == 0 and w13.data_ptr() % 16 == 0)
        if fused is None:
            fused = (can and self.use_gated and
                     self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated_supports(M, hidden, K) == 1)
        _need(can or not fused, "the fused form takes bfloat16, at most 64 rows, hidden % 64 == 0 and K % 8 == 0")
        if not fused:
            gate_up = self.linear(x, w13, partials_ok=True)
            return self.swiglu(gate_up if rs is None else rs.follow(gate_up), out_dtype=x.dtype)
        return self.gemm_gated(x, w13, rs)

    @_timed
    def gemm_gated(self, x: torch.Tensor, w13: torch.Tensor, rs: Optional[RowScaled] = None) -> torch.Tensor:
        """The one-kernel form of :meth:`linear_swiglu` (its caller has checked the sizes)."""
        M, K = x.shape
        hidden = w13.shape[0] // 2
        out = torch.empty((M, hidden), dtype=torch.bfloat16, device=x.device)
        rc = self._lib("gemm_tcgen05").tl_gemm_tcgen05_gated(
            _ptr(x), _ptr(w13), _ptr(out), M, hidden, K, *_scale_args(rs, M),
            ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05_gated")
        self.launches += 1
        return out

    def gemm_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """At most 64 rows of bfloat16 against a bfloat16 weight on the tcgen05 kernel.  Returns
        ``[M, N]`` in ``out_dtype`` when the weight's shape needs no K split, else float32 partial
        sums ``[splits, M, N]``."""
        _cuda_contig(x, "gemm input", torch.bfloat16)
        _cuda_contig(w, "gemm weight", torch.bfloat16)
        M, K = x.shape
        N = w.shape[0]
        _need(x.shape[1] == w.shape[1], "gemm_tcgen05: inner sizes differ")
        _need(1 <= M <= 64 and K % 8 == 0 and K >= 8, "gemm_tcgen05 takes 1..64 rows and K a multiple of 8")
        _need(out_dtype in _DT, f"gemm_tcgen05: output dtype {out_dtype} unsupported")
        lib = self._lib("gemm_tcgen05")
        splits = lib.tl_gemm_tcgen05_splits(M, N, K)
        f32 = out_dtype == torch.float32 or splits > 1
        out = torch.empty((splits, M, N), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
        rc = lib.tl_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), 1 if f32 else 0, M, N, K, splits,
                                 ctypes.c_void_p(self._status.data_ptr()), _stream())
        _check(rc, "gemm_tcgen05")
        self.launches += 1
        return out[0] if splits == 1 else out

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (call after a sync)."""
        code = int(self._status[0])
        if code != 0:
            self._status[0] = 0
            raise KernelError(f"a kernel gave up waiting (code {code}); its output is not valid")
        if self.debug:
            from .build import loaded_libraries
            kinds = {901: "a token id outside the vocabulary", 902: "a position outside the rotary table",
                     903: "a negative cache slot", 904: "a page outside the page tensor", 905: "a row outside the stream"}
            for name in loaded_libraries():
                code = self._lib(name).tl_debug_take()
                if code != 0:
                    raise KernelError(f"debug build: a kernel of {name} was given {kinds.get(code, 'a bad index')} "
                                      f"(code {code}); it skipped the access")

    def wait_selftest(self, limit_ms: float = 1.0) -> float:
        """Run a kernel whose only mbarrier wait nothing will ever satisfy, with a limit of
        ``limit_ms``.  It must give up and say so: :meth:`check_status` then raises, and the device
        stays usable.  Returns the milliseconds the wait took."""
        waited = torch.zeros(1, dtype=torch.int64, device="cuda")
        lib = self._lib("gemm_tcgen05")
        rc = lib.tl_wait_selftest(ctypes.c_void_p(self._status.data_ptr()), ctypes.c_ulonglong(int(limit_ms * 1e6)),
                                  _ptr(waited), _stream())
        _check(rc, "wait_selftest")
        torch.cuda.synchronize()
        return float(waited.item()) / 1e6

    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        _cuda_contig(x, "gemm input")
        _cuda_contig(w, "gemm weight")
        _need(x.shape[1] == w.shape[1] and x.dtype == w.dtype and x.dtype in _DT, "gemm_simt: operands disagree")
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
        rc = self._lib("gemm_simt").tl_gemm_simt(_ptr(x), _ptr(w), _ptr(out), _DT[x.dtype], _DT[out_dtype],
                                                M, N, K, _stream())
        _check(rc, "gemm_simt")
        self.launches += 1
        return out

    # -------------------------------------------------------------------- rope
    @_timed
    def rope_kv_write(self, qkv, positions: torch.Tensor, table: torch.Tensor, *,
                      n_heads: int, n_kv_heads: int, head_dim: int, interleaved: bool,
                      k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                      slot_mapping: Optional[torch.Tensor], page_size: int,
                      out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``qkv`` is ``[tokens, row]``, or float32 partial sums ``[splits, tokens, row]`` (then
        ``out_dtype`` is the dtype of q and of the pages), or a :class:`RowScaled` of either (every
        row is multiplied by its scale before it is rotated and stored)."""
        rs = qkv if isinstance(qkv, RowScaled) else None
        if rs is not None:
            qkv = rs.x
        _cuda_contig(qkv, "qkv")
        _cuda_contig(positions, "positions", torch.int32)
        _cuda_contig(table, "rotary table", torch.float32)
        splits = qkv.shape[0] if qkv.dim() == 3 else 1
        T = qkv.shape[-2]
        out_dtype = out_dtype or qkv.dtype
        _need(qkv.dim() in (2, 3) and qkv.shape[-1] == (n_heads + 2 * n_kv_heads) * head_dim and qkv.dtype in _DT,
              "qkv must be [tokens, (n_heads + 2 n_kv_heads) * head_dim]")
        _need(splits == 1 or qkv.dtype == torch.float32, "partial sums must be float32")
        _need(out_dtype in _DT and (out_dtype == qkv.dtype or qkv.dtype == torch.float32), "rope cannot widen bfloat16 input")
        _need(table.dim() == 3 and table.shape[1] == head_dim // 2 and table.shape[2] == 2,
              "rotary table must be [positions, head_dim / 2, 2]")
        _need(positions.numel() == T, "one position per token")
        if k_pages is not None:
            _cuda_contig(k_pages, "k_pages", out_dtype)
            _cuda_contig(v_pages, "v_pages", out_dtype)
            _cuda_contig(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages.shape[1:] == (n_kv_heads, page_size, head_dim) and v_pages.shape == k_pages.shape,
                  "pages must be [pages, n_kv_heads, page_size, head_dim]")
            _need(slot_mapping.numel() == T, "one cache slot per token")
        q = torch.empty((T, n_heads, head_dim), dtype=out_dtype, device=qkv.device)
        if k_pages is not None:
            self._debug_limit("rope", 0, k_pages.shape[0])
        rc = self._lib("rope").tl_rope_kv_write(
            _ptr(qkv), _DT[qkv.dtype], splits, _ptr(positions), _ptr(table),
            _ptr(slot_mapping if k_pages is not None else None),
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _DT[out_dtype], T, n_heads, n_kv_heads, head_dim,
            page_size, table.shape[0], 1 if interleaved else 0, *_scale_args(rs, T), _stream())
        _check(rc, "rope_kv_write")
        self.launches += 1
        return q

    # --------------------------------------------------------------- attention
    def _scratch(self, device: torch.device, floats: int, tag: str = "attention") -> Optional[torch.Tensor]:
        if floats <= 0:
            return None
        key = (device.index or 0, tag)
        buf = self._workspace.get(key)
        if buf is None or buf.numel() < floats:
            if buf is not None:
                self._retired.append(buf)      # a captured graph may still point into it
            buf = torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=device)
            self._workspace[key] = buf
        return buf

    @_timed
    def paged_attention(self, q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                        block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor, *,
                        n_seqs: int, max_q_len: int, max_kv_len: int, scale: float,
                        window: Optional[int], page_size: int, allow_split: bool = True,
                        impl: str = "auto", n_tokens: Optional[int] = None,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``impl``: ``"general"`` (CUDA cores, any supported size, both dtypes), ``"mma"`` (tensor
        cores, bfloat16, head_dim 16/32/64/128), ``"decode"`` (tensor cores fed by TMA, bfloat16,
        head_dim 64/128, steps whose requests bring one token or very few), ``"prefill"``
        (tcgen05 tensor cores with accumulators in tensor memory, bfloat16, head_dim 64/128, made
        for long portions; ``"prefill2"`` is its variant that multiplies probabilities as value +
        remainder) or ``"auto"`` (the most specialised kernel that applies).

        ``block_table``, ``q_start`` and ``kv_len`` may be slices that cover only some requests of
        the step (``q_start`` keeps counting tokens from the start of ``q``); ``n_tokens`` then
        bounds the rows those requests own (default: all of ``q``), and ``out`` lets several such
        calls fill one tensor.  ``allow_split``: False keeps every request's keys in one CTA, True lets
        the kernel split them as it sees fit; the decode kernel also takes a number of splits (above 1)."""
        _cuda_contig(q, "q")
        _cuda_contig(k_pages, "k_pages", q.dtype)
        _cuda_contig(v_pages, "v_pages", q.dtype)
        _cuda_contig(q_start, "q_start", torch.int32)
        _cuda_contig(kv_len, "kv_len", torch.int32)
        _need(block_table.is_cuda and block_table.dtype == torch.int32 and block_table.dim() == 2
              and block_table.stride(1) == 1, "block_table must be an int32 matrix with unit column stride")
        T, n_heads, head_dim = q.shape
        if n_tokens is not None:
            _need(0 < n_tokens <= T, "n_tokens must lie within q")
            T = int(n_tokens)
        if out is not None:
            _cuda_contig(out, "out", q.dtype)
            _need(out.shape == q.shape, "out must have q's shape")
        n_kv_heads = k_pages.shape[1]
        self.check_attention_sizes(n_heads, n_kv_heads, head_dim, q.dtype)
        _need(k_pages.shape[2] == page_size and k_pages.shape[3] == head_dim and v_pages.shape == k_pages.shape,
              "pages must be [pages, n_kv_heads, page_size, head_dim]")
        _need(block_table.shape[0] >= n_seqs and q_start.numel() >= n_seqs + 1 and kv_len.numel() >= n_seqs,
              "block_table, q_start and kv_len must cover every request of the step")
        _need(block_table.shape[1] * page_size >= max_kv_len, "block_table is too narrow for max_kv_len")
        _need(impl in ("auto", "general", "mma", "decode", "prefill", "prefill2"), f"unknown attention implementation {impl!r}")
        # "prefill2": the tcgen05 prefill kernel that multiplies probabilities as value + remainder
        parts = 2 if impl == "prefill2" else self.prefill_probability_parts
        if impl == "prefill2":
            impl = "prefill"
        mma_ok = q.dtype == torch.bfloat16 and head_dim in (16, 32, 64, 128)
        _need(impl != "mma" or mma_ok, "the tensor-core attention kernel takes bfloat16 and head_dim 16, 32, 64 or 128")
        use_mma = mma_ok and impl in ("auto", "mma")
        decode_ok = (q.dtype == torch.bfloat16 and impl in ("auto", "decode") and head_dim in (64, 128) and
                     self._lib("attention_decode").tl_attention_decode_supports(n_heads, n_kv_heads, head_dim,
                                                                                 page_size, max_q_len) == 1)
        _need(impl != "decode" or decode_ok, "the decode attention kernel takes bfloat16, head_dim 64 or 128, a "
              "power-of-two page size and requests whose rows fit one 16-row tile")
        n_splits = ctypes.c_int(0)
        floats = ctypes.c_longlong(0)
        if out is None:
            out = torch.empty_like(q)
        prefill_ok = (q.dtype == torch.bfloat16 and impl in ("auto", "prefill") and head_dim in (64, 128) and not decode_ok
                      and (impl == "prefill" or max_q_len >= self.PREFILL_MIN_Q) and
                      self._lib("attention_prefill").tl_attention_prefill_supports(n_heads, n_kv_heads, head_dim, page_size) == 1)
        _need(impl != "prefill" or prefill_ok, "the tcgen05 prefill attention kernel takes bfloat16, head_dim 64 or 128 "
              "and a power-of-two page size")
        if prefill_ok:
            lib = self._lib("attention_prefill")
            self._debug_limit("attention_prefill", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_prefill(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), ctypes.c_void_p(self._status.data_ptr()), ctypes.c_longlong(q.shape[0]),
                T, n_seqs, n_heads, n_kv_heads, head_dim, page_size, ctypes.c_longlong(k_pages.shape[0]), max_q_len,
                int(window or 0), ctypes.c_float(scale), parts, _stream())
            _check(rc, "paged_attention_prefill")
            self.launches += 1
            return out
        if decode_ok:
            lib = self._lib("attention_decode")
            rc = lib.tl_attention_decode_plan(T, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len,
                                              int(allow_split), ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_decode_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention_decode", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_decode(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), ctypes.c_void_p(self._status.data_ptr()), T, n_seqs,
                n_heads, n_kv_heads, head_dim, page_size, ctypes.c_longlong(k_pages.shape[0]), max_q_len, max_kv_len,
                int(window or 0), ctypes.c_float(scale), int(allow_split), _stream())
            _check(rc, "paged_attention_decode")
        elif use_mma:
            lib = self._lib("attention_mma")
            rc = lib.tl_attention_mma_plan(T, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len,
                                           1 if allow_split else 0, ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_mma_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention_mma", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention_mma(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), T, n_seqs, n_heads, n_kv_heads, head_dim,
                page_size, max_q_len, max_kv_len, int(window or 0), ctypes.c_float(scale),
                1 if allow_split else 0, _stream())
            _check(rc, "paged_attention_mma")
        else:
            lib = self._lib("attention")
            rc = lib.tl_attention_plan(T, n_seqs, n_heads, n_kv_heads, head_dim, max_q_len, max_kv_len,
                                       1 if allow_split else 0, ctypes.byref(n_splits), ctypes.byref(floats))
            _check(rc, "attention_plan")
            ws = self._scratch(q.device, floats.value)
            self._debug_limit("attention", 0, k_pages.shape[0])
            rc = lib.tl_paged_attention(
                _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(block_table), block_table.stride(0),
                _ptr(q_start), _ptr(kv_len), _ptr(ws), _DT[q.dtype], T, n_seqs, n_heads, n_kv_heads, head_dim,
                page_size, max_q_len, max_kv_len, int(window or 0), ctypes.c_float(scale),
                1 if allow_split else 0, _stream())
            _check(rc, "paged_attention")
        self.launches += 2 if n_splits.value > 1 else 1
        return out

    # ---------------------------------------------------------------- sampling
    @_timed
    def sample(self, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
               top_k: Optional[torch.Tensor] = None, row_keys: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next token of every row.  ``temperature`` (float32), ``top_k`` (int32) and
        ``row_keys`` (int64 holding the 64-bit key) are per row; without a temperature
        every row is greedy."""
        _need(logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1,
              "logits must be a float32 matrix on the GPU with unit column stride")
        n, vocab = logits.shape
        if temperature is not None:
            _cuda_contig(temperature, "temperature", torch.float32)
            _need(row_keys is not None, "sampling with a temperature needs row keys")
            _cuda_contig(row_keys, "row_keys", torch.int64)
            _need(temperature.numel() == n and row_keys.numel() == n, "one temperature and key per row")
        if top_k is not None:
            _cuda_contig(top_k, "top_k", torch.int32)
            _need(top_k.numel() == n, "one top_k per row")
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
        lib = self._lib("sampling")
        if top_k is None and vocab > 8192:
            # no rank filter: spread every row over many CTAs, then pick among their candidates
            lib.tl_sample_wide_scratch.restype = ctypes.c_longlong
            ws = self._scratch(logits.device, lib.tl_sample_wide_scratch(n, vocab), "sampling")
            rc = lib.tl_sample_wide(_ptr(logits), ctypes.c_longlong(logits.stride(0)), n, vocab, _ptr(temperature),
                                    _ptr(row_keys), _ptr(ws), _ptr(out), _stream())
            _check(rc, "sample_wide")
            self.launches += 2
            return out
        rc = lib.tl_sample(
            _ptr(logits), ctypes.c_longlong(logits.stride(0)), n, vocab, _ptr(temperature), _ptr(top_k),
            _ptr(row_keys), _ptr(out), _stream())
        _check(rc, "sample")
        self.launches += 1
        return out


def build_all() -> None:
    """Compile every kernel library (what ``__graft_entry__.build`` calls)."""
    build_libraries(ALL_LIBRARIES)
