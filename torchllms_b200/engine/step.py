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


class _StepBuffers:
    """Fixed-layout pinned host buffer and its device twin."""

    def __init__(self, cache: CacheManager, max_tokens: int, device: torch.device):
        B, T, NB, G = cache.max_num_seqs, max_tokens, cache.max_blocks, len(cache.groups)
        self.T, self.B, self.NB, self.G = T, B, NB, G
        off = 0
        self.sections = {}
        for name, n in (("token_ids", T), ("positions", T), ("seq_of_token", T), ("want_rows", T),
                        ("q_start", B + 1), ("kv_len", B), ("state_slot", B), ("fresh", B)):
            self.sections[name] = (off, n)
            off += n
        for g in range(G):
            self.sections[f"slot_mapping{g}"] = (off, T)
            off += T
        for g in range(G):
            self.sections[f"block_table{g}"] = (off, B * NB)
            off += B * NB
        self.total = off
        pin = device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        self.copied = torch.cuda.Event() if pin else None
        self._pending = False

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

    def upload(self, n_seqs: int) -> None:
        # everything up to the last block-table row in use, in one copy
        if self.G:
            off, _ = self.sections[f"block_table{self.G - 1}"]
            end = off + n_seqs * self.NB
        else:
            end = self.sections["fresh"][0] + self.B
        self.dev[:end].copy_(self.host[:end], non_blocking=True)
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
        # A step's launch shapes depend only on (tokens, requests, wanted rows, longest portion), never
        # on how long the requests have grown: the kernels read lengths and tables from the uploaded
        # buffers.  So a shape that keeps coming back (every decode step with the same number of
        # requests; every full prompt chunk) is recorded once into a CUDA graph and replayed.
        ops = model.ops
        self.use_graphs = bool(use_graphs and self.device.type == "cuda" and model.graph_safe
                               and getattr(ops, "graph_capturable", lambda d: False)(model.dtype))
        self._graphs = {}          # shape key -> (graph, logits buffer, launches)
        self._graph_seen = {}
        self.max_prompt_graphs = 16   # recorded shapes other than decode steps (each keeps its activations)
        self._graph_pool = None
        self.graph_replays = 0

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
        key = self._shape_key(ctx.n_tokens, ctx.n_seqs, ctx.n_want, ctx.max_q_len, ctx.n_decode)
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
    def _shape_key(n_tokens: int, n_seqs: int, n_want: int, max_q_len: int, n_decode: int):
        return (n_tokens, n_seqs, n_want, max_q_len, n_decode)

    def _replay(self, entry) -> Optional[torch.Tensor]:
        entry[0].replay()
        self.graph_replays += 1
        if hasattr(self.model.ops, "launches"):
            self.model.ops.launches += entry[2]
        return entry[1]

    def capture_decode_graphs(self, batch_sizes: Sequence[int]) -> int:
        """Record the decode-step graphs for these numbers of requests ahead of time, with
        throw-away requests (the cache must have room for one page each).  Returns how many
        graphs exist afterwards.  Without this a shape is recorded the second time it occurs."""
        if not self.use_graphs:
            return 0
        for b in sorted(set(int(x) for x in batch_sizes)):
            if b < 1 or b > self.cache.max_num_seqs or self._shape_key(b, b, b, 1, b) in self._graphs:
                continue
            if self.cache.n_live() + b > self.cache.max_num_seqs:
                continue
            handles = [self.claim() for _ in range(b)]
            try:
                for _ in range(3):          # one token each: eager, eager (first sight), recorded
                    self.step([StepEntry(h, [0]) for h in handles])
            except OutOfPages:
                pass
            finally:
                for h in handles:
                    self.release(h)
        torch.cuda.synchronize()
        return len(self._graphs)

    # --------------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch.  Returns float32 logits
        ``[n_wanted, vocab]`` on the device, rows in the order of the entries and
        of each entry's ``want``; ``None`` when nothing was wanted.

        Raises :class:`~torchllms_b200.cache.manager.OutOfPages` (nothing changed)
        when the pool cannot hold the new tokens."""
        if not entries:
            return None
        q_lens = [len(e.tokens) for e in entries]
        T, B = sum(q_lens), len(entries)
        if min(q_lens) <= 0:
            raise StepError("every entry of a step must bring at least one token")
        if T > self.max_step_tokens:
            raise StepError(f"a step may bring at most {self.max_step_tokens} tokens, got {T}")
        if B > self.cache.max_num_seqs:
            raise StepError(f"a step may hold at most {self.cache.max_num_seqs} requests, got {B}")
        flat = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=T)
        if flat.min() < 0 or flat.max() >= self.vocab_size:
            bad = int(flat[(flat < 0) | (flat >= self.vocab_size)][0])
            raise StepError(f"token id {bad} is outside the vocabulary (0..{self.vocab_size - 1})")
        want_rows: List[int] = []
        base = 0
        for e, n in zip(entries, q_lens):
            want = [n - 1] if e.want is None else list(e.want)
            for w in want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.handle}: wanted place {w} is outside its {n} tokens")
                want_rows.append(base + w)
            base += n

        cache = self.cache
        starts = cache.extend_many([(e.handle, n) for e, n in zip(entries, q_lens)])  # may raise OutOfPages
        buf = self._buf
        buf.wait_host_free()
        lens = np.asarray(q_lens, dtype=np.int64)
        first = np.asarray(starts, dtype=np.int64)
        q_start = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=q_start[1:])
        kv_lens = (first + lens).tolist()
        slots = [cache.slot(e.handle) for e in entries]
        # per token: which request it belongs to and its absolute position (no loop over requests)
        seq_of = np.repeat(np.arange(B, dtype=np.int64), lens)
        pos_all = np.arange(T, dtype=np.int64) - q_start[seq_of] + first[seq_of]
        buf.host_view("token_ids")[:T] = flat
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
                for e, s0 in zip(entries, starts):
                    cache.truncate(e.handle, s0)
                raise StepError("a token of this step falls on a page that was already given back")
            buf.host_view(f"slot_mapping{g}")[:T] = pages * page + pos_all % page
            buf.host_view(f"block_table{g}")[:B * buf.NB].reshape(B, buf.NB)[:] = rows
        buf.upload(B)

        decode_only = max(q_lens) == 1
        n_want = len(want_rows)
        n_decode = 0
        while n_decode < B and q_lens[n_decode] == 1:
            n_decode += 1
        try:
            recorded = self._graphs.get(self._shape_key(T, B, n_want, max(q_lens), n_decode)) if self.use_graphs else None
            if recorded is not None:
                # the graph reads the buffers uploaded above at their fixed addresses: nothing else to build
                logits = self._replay(recorded)
            else:
                ctx = StepContext(
                    n_tokens=T, n_seqs=B, n_want=n_want, max_q_len=max(q_lens), n_decode=n_decode,
                    # steps of short portions (where keys may be split over CTAs) plan for the longest
                    # sequence there can be, so that their launch shapes do not depend on the lengths
                    max_kv_len=self.max_len if max(q_lens) <= 16 else max(kv_lens),
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
            for e, s in zip(entries, starts):  # leave the cache as the step found it
                cache.truncate(e.handle, s)
            raise
        if self._has_window:
            for e in entries:
                cache.pass_window(e.handle)
        self.steps_run += 1
        self.tokens_run += T
        return logits
