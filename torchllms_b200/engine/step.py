"""The step function: one batch of (request, its next tokens) through the model.

Reference: ``Transformer.forward`` with a paged pool
(torchllms/models/networks.py:909-1049) builds per-forward index tensors
(``PagedBatchLayout``, torchllms/models/paged_kv.py:74-111, :486-617), derives
positions from the pool's lengths (:992-1015), runs the layers and keeps the
last row of each request (:1030-1045).  Its driver only ever builds whole-prompt
batches or one-token-per-request batches and requires every live request in
every forward (:984-990).  Here a step takes any subset of the live requests,
each with any number of next tokens (a portion of a prompt, or one decoded
token), runs exactly those tokens as one flat batch against the cache earlier
steps left, and returns float32 logits at the places asked for.

All index data of a step is packed on the host into one pinned int32 buffer
with a fixed layout and uploaded with a single copy; the device-side views
have fixed addresses, which is what CUDA-graph replay of decode steps needs.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages
from .model import Model


class StepError(ValueError):
    """A step was asked for that cannot run (bad token id, too many tokens, ...)."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and which of them want logits.

    ``want`` holds indices into ``tokens``; ``None`` means the last token only."""

    handle: int
    tokens: Sequence[int]
    want: Optional[Sequence[int]] = None


@dataclass
class PreparedStep:
    """What :meth:`Engine.prepare` decided: everything of a step but the token values."""

    handles: List[int]       # in batch order (see ``order``)
    q_lens: List[int]
    starts: List[int]        # each request's length before the step
    kv_lens: List[int]
    slots: List[int]
    n_want: int
    order: Optional[List[int]] = None   # batch place -> index among the caller's entries; None: as given


@dataclass
class StepContext:
    """What the parts see of a step (device tensors are views of one uploaded buffer)."""

    n_tokens: int
    n_seqs: int
    n_want: int
    max_q_len: int
    max_kv_len: int
    n_decode: int                # how many requests at the head of the batch bring exactly one token
    token_ids: torch.Tensor      # [T] int32
    positions: torch.Tensor      # [T] int32, absolute position of each token in its request
    seq_of_token: torch.Tensor   # [T] int32, index into the step's requests
    q_start: torch.Tensor        # [B + 1] int32, first token of each request in the flat batch
    kv_len: torch.Tensor         # [B] int32, request length after this step
    state_slot: torch.Tensor     # [B] int32, the request's slot (row of per-request state)
    fresh: torch.Tensor          # [B] int32, 1 where the portion starts at position 0
    want_rows: torch.Tensor      # [n_want] int32, flat indices of the tokens whose logits are wanted
    # host copies, for parts that plan on the host
    q_lens: List[int] = field(default_factory=list)
    kv_lens: List[int] = field(default_factory=list)
    slots: List[int] = field(default_factory=list)
    decode_kv_bound: int = 0     # the context length that the one-token rows of a mixed step plan their attention for


class _StepBuffers:
    """A pinned host buffer and its device twin.  A step's index data lie back to back, so that
    one copy of just the used part uploads them.  Where a section lies depends only on the step's
    numbers of tokens and requests: a recorded graph (there is one per such pair at least) finds
    its inputs at fixed addresses."""

    PER_TOKEN = ("token_ids", "positions", "seq_of_token", "want_rows", "token_src")   # token_ids stays first
    PER_SEQ = ("kv_len", "state_slot", "fresh")

    def __init__(self, cache: CacheManager, max_tokens: int, device: torch.device):
        B, T, NB, G = cache.max_num_seqs, max_tokens, cache.max_blocks, len(cache.groups)
        self.T, self.B, self.NB, self.G = T, B, NB, G
        self._layouts = {}
        self.sections, self.used = self._layout(T, B)
        self.total = self.used
        pin = device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event() if pin else None
        self._pending = False
        self.uploaded_bytes = 0

    def _layout(self, n_tokens: int, n_seqs: int):
        got = self._layouts.get((n_tokens, n_seqs))
        if got is None:
            sections, off = {}, 0
            sizes = [(name, n_tokens) for name in self.PER_TOKEN]
            sizes += [(f"slot_mapping{g}", n_tokens) for g in range(self.G)]
            sizes += [("q_start", n_seqs + 1)] + [(name, n_seqs) for name in self.PER_SEQ]
            sizes += [(f"block_table{g}", n_seqs * self.NB) for g in range(self.G)]
            for name, n in sizes:
                sections[name] = (off, n)
                off += -(-n // 4) * 4                     # every section starts on 16 bytes
            got = self._layouts[n_tokens, n_seqs] = (sections, off)
        return got

    def lay_out(self, n_tokens: int, n_seqs: int) -> None:
        """Place the sections for a step of this many tokens and requests."""
        self.sections, self.used = self._layout(n_tokens, n_seqs)

    def host_view(self, name: str) -> np.ndarray:
        off, n = self.sections[name]
        return self.host_np[off:off + n]

    def dev_view(self, name: str, n: Optional[int] = None) -> torch.Tensor:
        off, full = self.sections[name]
        return self.dev[off:off + (full if n is None else n)]

    def wait_host_free(self) -> None:
        if self._pending and self.copied is not None:
            self.copied.synchronize()
        self._pending = False

    def upload(self, skip_tokens: bool = False) -> None:
        # the sections in use, in one copy; the token ids (the first section) stay behind when the
        # device has them already
        start, end = (self.sections["positions"][0] if skip_tokens else 0), self.used
        self.uploaded_bytes = 4 * (end - start)
        self.dev[start:end].copy_(self.host[start:end], non_blocking=True)
        if self.copied is not None:
            self.copied.record()
            self._pending = True


class Engine:
    """A model, its cache, and the step function over them."""

    def __init__(self, model: Model, *, page_size: int = 16, pool_tokens: int, max_num_seqs: int = 64,
                 max_len: Optional[int] = None, max_step_tokens: int = 8192, use_graphs: bool = True):
        self.model = model
        self.device = model.device
        self.max_len = int(max_len or model.max_positions)
        if self.max_len > model.max_positions:
            raise StepError(f"max_len {self.max_len} exceeds the model's position table ({model.max_positions})")
        self.max_step_tokens = int(max_step_tokens)
        self.cache = CacheManager(model.run_needs(), page_size=page_size, pool_tokens=pool_tokens,
                                  max_num_seqs=max_num_seqs, max_len=self.max_len, dtype=model.dtype,
                                  device=self.device, max_step_tokens=self.max_step_tokens)
        self._buf = _StepBuffers(self.cache, self.max_step_tokens, self.device)
        self._has_window = any(g.need.kind == "window" for g in self.cache.groups)
        self.vocab_size = model.spec.vocab_size
        self.steps_run = 0
        self.tokens_run = 0
        # A step's launch shapes depend only on (tokens, requests, wanted rows, longest portion) and, for
        # steps of short portions, on a coarse bound of the longest context (a power of two: it decides
        # over how many CTAs the keys are split), never on the exact lengths: the kernels read lengths
        # and tables from the uploaded buffers.  So a shape that keeps coming back (every decode step
        # with the same number of requests; every full prompt chunk) is recorded once into a CUDA graph
        # and replayed.
        ops = model.ops
        self.use_graphs = bool(use_graphs and self.device.type == "cuda" and model.graph_safe
                               and getattr(ops, "graph_capturable", lambda d: False)(model.dtype))
        self._graphs = {}          # shape key -> (graph, logits buffer, launches)
        self._graph_seen = {}
        self.max_prompt_graphs = 16   # recorded shapes other than decode steps (each keeps its activations)
        self._graph_pool = None
        self.graph_replays = 0
        self._forced_bound: Optional[int] = None      # capture_decode_graphs: record for this context bound
        # TORCHLLMS_B200_DEBUG=1: range-check every index array of a step on the host before it is uploaded
        self.debug = os.environ.get("TORCHLLMS_B200_DEBUG", "") not in ("", "0")

    # ----------------------------------------------------------------- requests
    def claim(self) -> int:
        return self.cache.claim()

    def release(self, handle: int) -> None:
        self.cache.release(handle)

    def can_run(self, wants: Sequence[Tuple[int, int]]) -> bool:
        return self.cache.can_extend(wants)

    def _forward_graphed(self, ctx: StepContext, views) -> Optional[torch.Tensor]:
        """A decode shape is recorded the second time it occurs, any other shape the third time
        (while fewer than ``max_prompt_graphs`` of those exist); later steps replay.  The logits
        buffer of a shape is reused: its contents hold until the next step of that shape."""
        key = self._shape_key(ctx.n_tokens, ctx.n_seqs, ctx.n_want, ctx.max_q_len, ctx.n_decode,
                              ctx.max_kv_len if ctx.max_q_len <= 16 else 0, ctx.decode_kv_bound)
        entry = self._graphs.get(key)
        if entry is None:
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            decode = ctx.max_q_len == 1
            full = (not decode) and sum(1 for k in self._graphs if k[3] != 1) >= self.max_prompt_graphs
            if seen < (1 if decode else 2) or full:
                return self.model.forward(ctx, views)          # eager: loads libraries, sizes scratch
            ops = self.model.ops
            before = getattr(ops, "launches", 0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                out = self.model.forward(ctx, views)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, out, getattr(ops, "launches", 0) - before)
            self._graphs[key] = entry
            if hasattr(ops, "launches"):
                ops.launches = before
        return self._replay(entry)

    @staticmethod
    def _shape_key(n_tokens: int, n_seqs: int, n_want: int, max_q_len: int, n_decode: int, kv_bound: int,
                   decode_bound: int = 0):
        return (n_tokens, n_seqs, n_want, max_q_len, n_decode, kv_bound, decode_bound)

    BOUND_BELOW = 16     # steps of fewer requests plan for a bound of their longest context, others for max_len

    def kv_bound(self, longest: int, n_seqs: int) -> int:
        """The context length that a step of short portions plans its attention for.  With few
        requests the kernel splits each one's keys over many CTAs, as many as the length allows:
        such steps plan for the power of two (at least 1,024, at most ``max_len``) that holds their
        longest context.  With ``BOUND_BELOW`` requests or more the requests themselves fill the GPU
        and the plan does not depend on the length: they plan for ``max_len``."""
        if n_seqs >= self.BOUND_BELOW:
            return self.max_len
        b = 1024
        while b < longest:
            b *= 2
        return min(b, self.max_len)

    def kv_bounds(self, n_seqs: int) -> List[int]:
        """Every value ``kv_bound`` can take for this many requests."""
        return sorted(set(self.kv_bound(1 << k, n_seqs) for k in range(10, max(self.max_len, 1024).bit_length() + 1)))

    def _replay(self, entry) -> Optional[torch.Tensor]:
        entry[0].replay()
        self.graph_replays += 1
        if hasattr(self.model.ops, "launches"):
            self.model.ops.launches += entry[2]
        return entry[1]

    def capture_decode_graphs(self, batch_sizes: Sequence[int], context_lengths: Optional[Sequence[int]] = None) -> int:
        """Record the decode-step graphs for these numbers of requests ahead of time, with throw-away
        requests (the cache must have room for one page each): for every context bound that steps of
        so many requests can plan for (``kv_bounds``), or only for those of the given context
        lengths.  Returns how many graphs exist afterwards.  Without this a shape is recorded the
        second time it occurs."""
        if not self.use_graphs:
            return 0
        for b in sorted(set(int(x) for x in batch_sizes)):
            bounds = self.kv_bounds(b) if context_lengths is None else sorted(set(self.kv_bound(int(n), b) for n in context_lengths))
            for bound in bounds:
                if b < 1 or b > self.cache.max_num_seqs or self._shape_key(b, b, b, 1, b, bound) in self._graphs:
                    continue
                if self.cache.n_live() + b > self.cache.max_num_seqs:
                    continue
                handles = [self.claim() for _ in range(b)]
                self._forced_bound = bound
                try:
                    for _ in range(3):          # one token each: eager, eager (first sight), recorded
                        self.step([StepEntry(h, [0]) for h in handles])
                except OutOfPages:
                    pass
                finally:
                    self._forced_bound = None
                    for h in handles:
                        self.release(h)
        torch.cuda.synchronize()
        return len(self._graphs)

    # --------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch.  Returns float32 logits
        ``[n_wanted, vocab]`` on the device, rows in the order of the entries and
        of each entry's ``want``; ``None`` when nothing was wanted.  (With CUDA graphs
        on, the tensor is a buffer the next step of the same shape writes again.)

        Raises :class:`~torchllms_b200.cache.manager.OutOfPages` (nothing changed)
        when the pool cannot hold the new tokens."""
        if not entries:
            return None
        prepared = self.prepare([(e.handle, len(e.tokens), e.want) for e in entries])
        return self.run_prepared(prepared, [t for e in entries for t in e.tokens])

    def prepare(self, shape: Sequence[Tuple[int, int, Optional[Sequence[int]]]]) -> "PreparedStep":
        """The host half of a step that does not need the token values: ``shape`` holds
        ``(handle, n_tokens, want)`` per request.  Grows the cache and packs positions, cache
        slots, block tables and wanted rows into the pinned buffer.  A scheduler may call this for
        the next step while the device still runs the current one, then :meth:`run_prepared` once
        the tokens are known, or :meth:`discard` if the step will not happen after all.  Only one
        prepared step can exist at a time."""
        shape = [(h, int(n), w) for h, n, w in shape]
        T, B = sum(n for _h, n, _w in shape), len(shape)
        if B == 0 or min(n for _h, n, _w in shape) <= 0:
            raise StepError("every entry of a step must bring at least one token")
        if T > self.max_step_tokens:
            raise StepError(f"a step may bring at most {self.max_step_tokens} tokens, got {T}")
        if B > self.cache.max_num_seqs:
            raise StepError(f"a step may hold at most {self.cache.max_num_seqs} requests, got {B}")
        for h, n, want in shape:
            for w in (want or ()):
                if not 0 <= w < n:
                    raise StepError(f"request {h}: wanted place {w} is outside its {n} tokens")
            if want is not None and len(set(want)) != len(want):
                raise StepError(f"request {h}: a place is wanted twice")
        # Inside the batch, requests that bring one token stand before those that bring more (each kind
        # in the caller's order): the mixer sends the two kinds to kernels made for them.  The wanted
        # rows keep the caller's order, so nothing of this shows outside.
        order = sorted(range(B), key=lambda i: shape[i][1] != 1)
        identity = order == list(range(B))
        handles = [shape[i][0] for i in order]
        q_lens = [shape[i][1] for i in order]
        base_of = [0] * B                       # caller's entry -> its first row in the batch
        base = 0
        for i in order:
            base_of[i] = base
            base += shape[i][1]
        want_rows: List[int] = []
        for i, (_h, n, want) in enumerate(shape):
            want_rows += [base_of[i] + w for w in ([n - 1] if want is None else want)]

        cache = self.cache
        starts = cache.extend_many(list(zip(handles, q_lens)))  # may raise OutOfPages
        try:
            buf = self._buf
            buf.wait_host_free()
            buf.lay_out(T, B)
            lens = np.asarray(q_lens, dtype=np.int64)
            first = np.asarray(starts, dtype=np.int64)
            q_start = np.zeros(B + 1, dtype=np.int64)
            np.cumsum(lens, out=q_start[1:])
            kv_lens = (first + lens).tolist()
            slots = [cache.slot(h) for h in handles]
            # per token: which request it belongs to and its absolute position (no loop over requests)
            seq_of = np.repeat(np.arange(B, dtype=np.int64), lens)
            pos_all = np.arange(T, dtype=np.int64) - q_start[seq_of] + first[seq_of]
            buf.host_view("positions")[:T] = pos_all
            buf.host_view("seq_of_token")[:T] = seq_of
            buf.host_view("q_start")[:B + 1] = q_start
            buf.host_view("kv_len")[:B] = kv_lens
            buf.host_view("state_slot")[:B] = slots
            buf.host_view("fresh")[:B] = first == 0
            buf.host_view("want_rows")[:len(want_rows)] = want_rows
            page = cache.page_size
            for g in range(len(cache.groups)):
                rows = cache.block_table_rows(g, slots)                       # [B, max_blocks]
                pages = rows[seq_of, pos_all // page]
                if (pages < 0).any():
                    raise StepError("a token of this step falls on a page that was already given back")
                buf.host_view(f"slot_mapping{g}")[:T] = pages * page + pos_all % page
                buf.host_view(f"block_table{g}")[:B * buf.NB].reshape(B, buf.NB)[:] = rows
            if self.debug:
                self._check_packed(T, B, len(want_rows))
        except BaseException:
            for h, s0 in zip(handles, starts):      # whatever went wrong, the cache is as the step found it
                cache.truncate(h, s0)
            raise
        return PreparedStep(handles, q_lens, starts, kv_lens, slots, len(want_rows), None if identity else order)

    @staticmethod
    def _in_batch_order(prepared: "PreparedStep", per_token: Sequence) -> Sequence:
        """Per-token values given in the caller's order of entries, in the batch's order."""
        if prepared.order is None:
            return per_token
        B = len(prepared.order)
        given_len = [0] * B
        for place, i in enumerate(prepared.order):
            given_len[i] = prepared.q_lens[place]
        offset = [0] * (B + 1)
        for i in range(B):
            offset[i + 1] = offset[i] + given_len[i]
        out: list = []
        for i in prepared.order:
            out.extend(per_token[offset[i]:offset[i + 1]])
        return out

    def _check_packed(self, T: int, B: int, n_want: int) -> None:
        """Debug mode: every index the kernels will trust lies where it must (the reference checks
        its layout on the host too, torchllms/models/paged_kv.py:797-843)."""
        buf, cache = self._buf, self.cache

        def within(name: str, values: np.ndarray, lo: int, hi: int) -> None:
            bad = np.nonzero((values < lo) | (values >= hi))[0]
            if bad.size:
                raise StepError(f"debug check: {name}[{int(bad[0])}] = {int(values[bad[0]])} is outside {lo}..{hi - 1}")

        within("positions", buf.host_view("positions")[:T], 0, self.max_len)
        within("seq_of_token", buf.host_view("seq_of_token")[:T], 0, B)
        within("want_rows", buf.host_view("want_rows")[:n_want], 0, T)
        within("state_slot", buf.host_view("state_slot")[:B], 0, cache.max_num_seqs)
        within("kv_len", buf.host_view("kv_len")[:B], 1, self.max_len + 1)
        q_start = buf.host_view("q_start")[:B + 1]
        if q_start[0] != 0 or q_start[B] != T or (np.diff(q_start) <= 0).any():
            raise StepError(f"debug check: q_start {q_start.tolist()} does not cut {T} tokens into {B} portions")
        for g, group in enumerate(cache.groups):
            n_pages = group.allocator.n_pages
            within(f"slot_mapping{g}", buf.host_view(f"slot_mapping{g}")[:T], 0, n_pages * cache.page_size)
            table = buf.host_view(f"block_table{g}")[:B * buf.NB]
            within(f"block_table{g}", table, -1, n_pages)      # -1: no page (never allocated, or given back)

    def discard(self, prepared: "PreparedStep") -> None:
        """Undo :meth:`prepare`: the cache is as it was before (requests released meanwhile are skipped)."""
        live = set(self.cache.live_handles())
        for h, s0 in zip(prepared.handles, prepared.starts):
            if h in live:
                self.cache.truncate(h, s0)

    def run_prepared(self, prepared: "PreparedStep", tokens, rows: Optional[Sequence[int]] = None) -> Optional[torch.Tensor]:
        """The device half: upload the packed buffer with these token ids and run the model.
        ``tokens`` is a list of ids, or an int32 tensor on the device (ids the sampler has just
        written and the host has not seen yet: they are taken as they are); with ``rows``, the
        step's ids are ``tokens[rows]``, gathered on the device.  Nothing here waits for the device."""
        q_lens, starts, kv_lens, slots = prepared.q_lens, prepared.starts, prepared.kv_lens, prepared.slots
        handles = prepared.handles
        T, B, n_want = sum(q_lens), len(q_lens), prepared.n_want
        cache, buf = self.cache, self._buf
        buf.lay_out(T, B)
        try:
            if isinstance(tokens, torch.Tensor):
                if tokens.dtype != torch.int32 or tokens.device != buf.dev.device or tokens.dim() != 1:
                    raise StepError("token ids on the device must be an int32 vector on the engine's device")
                rows = list(range(T)) if rows is None else list(rows)
                if len(rows) != T or min(rows) < 0 or max(rows) >= tokens.shape[0]:
                    raise StepError(f"the prepared step holds {T} tokens; rows {rows} of {tokens.shape[0]} ids do not give them")
                rows = self._in_batch_order(prepared, rows)
                buf.host_view("token_src")[:T] = rows      # the gather's index rides in the step's one upload
                buf.upload(skip_tokens=True)
                torch.index_select(tokens, 0, buf.dev_view("token_src", T), out=buf.dev_view("token_ids", T))
            elif len(tokens) != T:
                raise StepError(f"the prepared step holds {T} tokens, got {len(tokens)}")
            else:
                flat = np.asarray(self._in_batch_order(prepared, tokens), dtype=np.int64)
                if flat.min() < 0 or flat.max() >= self.vocab_size:
                    bad = int(flat[(flat < 0) | (flat >= self.vocab_size)][0])
                    raise StepError(f"token id {bad} is outside the vocabulary (0..{self.vocab_size - 1})")
                buf.host_view("token_ids")[:T] = flat
                buf.upload()
            max_q = max(q_lens)
            n_decode = 0
            while n_decode < B and q_lens[n_decode] == 1:
                n_decode += 1
            # steps of short portions (where keys may be split over CTAs) plan for a coarse bound of the
            # longest context, so that their launch shapes change only when a request outgrows it
            short = max_q <= 16
            bound = (self._forced_bound or self.kv_bound(max(kv_lens), B)) if short else 0
            # a mixed step's one-token rows go to the decode kernel apart from the portions: their own bound
            decode_bound = self.kv_bound(max(kv_lens[:n_decode]), n_decode) if 0 < n_decode < B else 0
            recorded = (self._graphs.get(self._shape_key(T, B, n_want, max_q, n_decode, bound, decode_bound))
                        if self.use_graphs else None)
            if recorded is not None:
                # the graph reads the buffers uploaded above at their fixed addresses: nothing else to build
                logits = self._replay(recorded)
            else:
                ctx = StepContext(
                    n_tokens=T, n_seqs=B, n_want=n_want, max_q_len=max_q, n_decode=n_decode,
                    max_kv_len=bound if short else max(kv_lens), decode_kv_bound=decode_bound,
                    token_ids=buf.dev_view("token_ids", T), positions=buf.dev_view("positions", T),
                    seq_of_token=buf.dev_view("seq_of_token", T), q_start=buf.dev_view("q_start", B + 1),
                    kv_len=buf.dev_view("kv_len", B), state_slot=buf.dev_view("state_slot", B),
                    fresh=buf.dev_view("fresh", B), want_rows=buf.dev_view("want_rows", n_want),
                    q_lens=q_lens, kv_lens=kv_lens, slots=slots)
                block_tables = [buf.dev_view(f"block_table{g}", B * buf.NB).view(B, buf.NB) for g in range(len(cache.groups))]
                slot_maps = [buf.dev_view(f"slot_mapping{g}", T) for g in range(len(cache.groups))]
                views = [cache.run_view(i, block_tables, slot_maps) for i in range(cache.n_runs)]
                if self.use_graphs:
                    logits = self._forward_graphed(ctx, views)
                else:
                    logits = self.model.forward(ctx, views)
        except BaseException:
            for h, s0 in zip(handles, starts):  # leave the cache as the step found it
                cache.truncate(h, s0)
            raise
        if self._has_window:
            for h in handles:
                cache.pass_window(h)
        self.steps_run += 1
        self.tokens_run += T
        return logits
