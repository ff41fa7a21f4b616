"""The cache manager: paged keys and values, block tables, and state slots.

Reference: ``PagedKVPool`` (torchllms/models/paged_kv.py:119-843).  Kept from
it: pages of ``page_size`` tokens, a free list used as a stack so that the page
freed last is used again first (:226, :290, :326-327), a reference count per
page (:225), a block table and a length per live request (:230-231) with
``len(pages) == ceil(length / page_size)`` (:129-130), lazy growth (:332-350),
handles that are never used twice (:271-281) and an invariant checker
(:797-843).  Different from it: growth is all-or-nothing over a whole batch;
runs of layers are sorted into *groups* by what they need (all keys, or a
window of them), each group with pages and block tables of its own, a window
group giving pages back once the window has passed them; and every live
request also owns a dense *slot* that indexes fixed-size state rows and the
engine's static per-request buffers.

Page tensors are laid out ``[run, page, kv_head, slot_in_page, head_dim]`` so
that one head's part of a page is one contiguous tile.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheNeed, StateNeed


class OutOfPages(RuntimeError):
    """The pool cannot hold the tokens that were asked for; nothing was allocated."""


class CacheError(RuntimeError):
    """Misuse of the cache manager (unknown handle, double release, ...)."""


FREED = -1  # block-table entry of a page that was given back (window) or never allocated


class PageAllocator:
    """Free list (a stack) and reference counts of one group's pages."""

    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = int(n_pages)
        # Pop from the end: page 0 goes out first, a page given back goes out next.
        self._free: List[int] = list(range(self.n_pages - 1, -1, -1))
        self._refs = np.zeros(self.n_pages, dtype=np.int32)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.n_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._refs[p] = 1
        return pages

    def share(self, page: int) -> None:
        if self._refs[page] <= 0:
            raise CacheError(f"page {page} is free and cannot be shared")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        if not 0 <= page < self.n_pages or self._refs[page] <= 0:
            raise CacheError(f"page {page} released while free (freed twice?)")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return int(self._refs[page])

    def free_pages(self) -> List[int]:
        return list(self._free)


@dataclass
class _Request:
    handle: int
    slot: int
    length: int = 0
    # per group: logical block -> page id (FREED where given back)
    blocks: List[List[int]] = field(default_factory=list)
    # per group: first logical block that still holds a page
    first_block: List[int] = field(default_factory=list)


@dataclass
class RunCacheView:
    """What one run of a mixer sees of the cache during a step."""

    k_pages: Optional[torch.Tensor]      # [pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # [n_seqs, max_blocks] int32, FREED where no page
    slot_mapping: Optional[torch.Tensor]  # [n_tokens] int32: page * page_size + offset
    page_size: int
    writes: bool                         # False for a run that reads another run's cache
    state: Optional[torch.Tensor]        # [max_num_seqs, *shape]; rows indexed by ctx.state_slot
    window: Optional[int] = None


class CacheGroup:
    """Runs with one and the same :class:`CacheNeed`: one allocator, one block table per request."""

    def __init__(self, index: int, need: CacheNeed, runs: List[int], n_pages: int, page_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.index = index
        self.need = need
        self.runs = list(runs)
        self.page_size = page_size
        self.allocator = PageAllocator(n_pages)
        shape = (len(runs), n_pages, need.n_kv_heads, page_size, need.head_dim)
        self.k_pages = torch.zeros(shape, dtype=dtype, device=device)
        self.v_pages = torch.zeros(shape, dtype=dtype, device=device)
        self.run_index = {run: i for i, run in enumerate(self.runs)}

    def bytes(self) -> int:
        return 2 * self.k_pages.numel() * self.k_pages.element_size()


class CacheManager:
    """Pages, block tables and state slots for every run of a model.

    ``run_needs[i]`` is ``(cache_need, state_need, cache_of)`` of run ``i`` in
    the model's run order; a run with ``cache_of = j`` owns no pages and reads
    run ``j``'s.  ``pool_tokens`` is how many tokens all live requests may hold
    together (each request's count rounded up to whole pages).
    """

    def __init__(self, run_needs: Sequence[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]],
                 *, page_size: int, pool_tokens: int, max_num_seqs: int, max_len: int,
                 dtype: torch.dtype, device, max_step_tokens: Optional[int] = None):
        if page_size <= 0 or pool_tokens <= 0 or max_num_seqs <= 0 or max_len <= 0:
            raise ValueError("page_size, pool_tokens, max_num_seqs and max_len must be positive")
        self.page_size = int(page_size)
        self.max_num_seqs = int(max_num_seqs)
        self.max_len = int(max_len)
        self.max_blocks = -(-self.max_len // self.page_size)
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_runs = len(run_needs)
        full_pages = -(-int(pool_tokens) // self.page_size)

        # ---- groups of runs by need
        self.groups: List[CacheGroup] = []
        self._group_of_run: List[Optional[int]] = [None] * self.n_runs
        self._owner_of_run: List[Optional[int]] = [None] * self.n_runs
        by_need: Dict[CacheNeed, List[int]] = {}
        for i, (need, _state, cache_of) in enumerate(run_needs):
            if cache_of is not None:
                continue
            if need is not None:
                by_need.setdefault(need, []).append(i)
        for need, runs in by_need.items():
            n_pages = full_pages
            if need.kind == "window":
                step = max_step_tokens if max_step_tokens is not None else self.max_len
                per_req = -(-(need.window + step) // self.page_size) + 1
                n_pages = min(full_pages, self.max_num_seqs * per_req)
            g = CacheGroup(len(self.groups), need, runs, n_pages, self.page_size, dtype, self.device)
            self.groups.append(g)
            for r in runs:
                self._group_of_run[r] = g.index
                self._owner_of_run[r] = r
        for i, (need, _state, cache_of) in enumerate(run_needs):
            if cache_of is not None:
                if self._group_of_run[cache_of] is None:
                    raise ValueError(f"run {i} reads the cache of run {cache_of}, which has none")
                donor = run_needs[cache_of][0]
                if need is not None and (need.n_kv_heads, need.head_dim) != (donor.n_kv_heads, donor.head_dim):
                    raise ValueError(f"run {i} cannot read run {cache_of}'s cache: head layout differs")
                self._group_of_run[i] = self._group_of_run[cache_of]
                self._owner_of_run[i] = cache_of

        # ---- state rows, one tensor per run that wants state
        self.state: List[Optional[torch.Tensor]] = []
        for _need, state, _ in run_needs:
            if state is None:
                self.state.append(None)
            else:
                self.state.append(torch.zeros((self.max_num_seqs, *state.shape), dtype=state.dtype,
                                              device=self.device))

        # ---- requests
        self._free_slots: List[int] = list(range(self.max_num_seqs - 1, -1, -1))
        self._requests: Dict[int, _Request] = {}
        self._next_handle = 0
        # host block tables, one per group, indexed by slot
        self._tables = [np.full((self.max_num_seqs, self.max_blocks), FREED, dtype=np.int32)
                        for _ in self.groups]

    # ------------------------------------------------------------------ queries
    def n_live(self) -> int:
        return len(self._requests)

    def live_handles(self) -> List[int]:
        return list(self._requests)

    def length(self, handle: int) -> int:
        return self._req(handle).length

    def slot(self, handle: int) -> int:
        return self._req(handle).slot

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.n_free

    def pages_of(self, handle: int, group: int = 0) -> List[int]:
        return list(self._req(handle).blocks[group])

    def block_table_rows(self, group: int, slots: Sequence[int]) -> np.ndarray:
        return self._tables[group][np.asarray(slots, dtype=np.int64)]

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)

    def _req(self, handle: int) -> _Request:
        try:
            return self._requests[handle]
        except KeyError:
            raise CacheError(f"request handle {handle} is not live") from None

    # ------------------------------------------------------------ claim / free
    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def claim(self) -> int:
        """A new, empty request: a fresh handle, a slot, zeroed state rows."""
        if not self._free_slots:
            raise CacheError(f"all {self.max_num_seqs} request slots are in use")
        slot = self._free_slots.pop()
        handle = self._next_handle
        self._next_handle += 1
        self._requests[handle] = _Request(handle, slot, 0, [[] for _ in self.groups], [0 for _ in self.groups])
        for s in self.state:
            if s is not None:
                s[slot].zero_()
        return handle

    def release(self, handle: int) -> None:
        """The request is finished (or pre-empted): every page and its slot are given back."""
        req = self._req(handle)
        for g, blocks in zip(self.groups, req.blocks):
            for p in blocks:
                if p != FREED:
                    g.allocator.release(p)
            self._tables[g.index][req.slot, :len(blocks)] = FREED
        del self._requests[handle]
        self._free_slots.append(req.slot)

    # ------------------------------------------------------------------ growth
    def _blocks_wanted(self, req: _Request, group: int, n_new: int) -> int:
        return max(0, -(-(req.length + n_new) // self.page_size) - len(req.blocks[group]))

    def can_extend(self, wants: Iterable[Tuple[int, int]]) -> bool:
        """Would :meth:`extend_many` succeed for these ``(handle, n_new_tokens)``?"""
        need = [0] * len(self.groups)
        for handle, n in wants:
            req = self._req(handle)
            if req.length + n > self.max_len:
                return False
            for gi in range(len(self.groups)):
                need[gi] += self._blocks_wanted(req, gi, n)
        return all(need[gi] <= g.allocator.n_free for gi, g in enumerate(self.groups))

    def room_for(self, handle: int, others: Iterable[Tuple[int, int]] = ()) -> int:
        """How many more tokens this request could take after ``others`` took theirs."""
        req = self._req(handle)
        others = list(others)
        room = self.max_len - req.length
        for gi, g in enumerate(self.groups):
            free = g.allocator.n_free - sum(self._blocks_wanted(self._req(h), gi, n) for h, n in others)
            room = min(room, (len(req.blocks[gi]) + max(free, 0)) * self.page_size - req.length)
        return max(room, 0)

    def extend_many(self, wants: Sequence[Tuple[int, int]]) -> List[int]:
        """Make room for ``n`` more tokens of each request, all or nothing.

        Returns each request's length before the call (the position of its
        first new token) and advances the lengths."""
        seen = set()
        for handle, n in wants:
            if handle in seen:
                raise CacheError(f"request handle {handle} appears twice in one batch")
            seen.add(handle)
            if n <= 0:
                raise CacheError(f"request {handle}: a step must bring at least one token")
            req = self._req(handle)
            if req.length + n > self.max_len:
                raise CacheError(
                    f"request {handle}: {req.length} + {n} tokens exceed the longest sequence ({self.max_len})")
        need = [sum(self._blocks_wanted(self._req(h), gi, n) for h, n in wants) for gi in range(len(self.groups))]
        for gi, g in enumerate(self.groups):
            if need[gi] > g.allocator.n_free:
                raise OutOfPages(
                    f"group {gi} ({g.need.kind}): {need[gi]} pages wanted, {g.allocator.n_free} of "
                    f"{g.allocator.n_pages} free")
        starts = []
        for handle, n in wants:
            req = self._req(handle)
            for gi, g in enumerate(self.groups):
                k = self._blocks_wanted(req, gi, n)
                if k:
                    new = g.allocator.alloc(k)
                    lo = len(req.blocks[gi])
                    req.blocks[gi].extend(new)
                    self._tables[gi][req.slot, lo:lo + k] = new
            starts.append(req.length)
            req.length += n
        return starts

    def pass_window(self, handle: int) -> int:
        """After a step: give back the pages of window groups that no later query can see.

        A query at position ``p`` of a window ``w`` reads keys ``p - w + 1 .. p``;
        the next query sits at ``length``.  Returns how many pages were freed."""
        req = self._req(handle)
        freed = 0
        for gi, g in enumerate(self.groups):
            if g.need.kind != "window":
                continue
            first_needed = req.length - g.need.window + 1
            last_dead_block = first_needed // self.page_size if first_needed > 0 else 0
            for b in range(req.first_block[gi], min(last_dead_block, len(req.blocks[gi]))):
                p = req.blocks[gi][b]
                if p != FREED:
                    g.allocator.release(p)
                    req.blocks[gi][b] = FREED
                    self._tables[gi][req.slot, b] = FREED
                    freed += 1
            req.first_block[gi] = max(req.first_block[gi], min(last_dead_block, len(req.blocks[gi])))
        return freed

    def truncate(self, handle: int, new_length: int) -> None:
        """Shorten a request; trailing pages go back (torchllms/models/paged_kv.py:367-405)."""
        req = self._req(handle)
        if not 0 <= new_length <= req.length:
            raise CacheError(f"request {handle}: cannot truncate {req.length} tokens to {new_length}")
        keep = -(-new_length // self.page_size)
        for gi, g in enumerate(self.groups):       # check every group before touching any
            if g.need.kind == "window" and req.first_block[gi] > 0:
                first_needed = new_length - g.need.window + 1
                if first_needed < req.first_block[gi] * self.page_size:
                    raise CacheError(
                        f"request {handle}: truncating to {new_length} would need keys that window "
                        f"group {gi} has already given back")
        for gi, g in enumerate(self.groups):
            while len(req.blocks[gi]) > keep:
                p = req.blocks[gi].pop()
                if p != FREED:
                    g.allocator.release(p)
                self._tables[gi][req.slot, len(req.blocks[gi])] = FREED
            req.first_block[gi] = min(req.first_block[gi], len(req.blocks[gi]))
        req.length = new_length

    # ---------------------------------------------------------- step-side views
    def slot_mapping(self, group: int, handle: int, start: int, n: int) -> np.ndarray:
        """Flat cache position ``page * page_size + offset`` of tokens ``start .. start + n - 1``."""
        req = self._req(handle)
        pos = np.arange(start, start + n, dtype=np.int64)
        pages = np.asarray(req.blocks[group], dtype=np.int64)[pos // self.page_size]
        if (pages == FREED).any():
            raise CacheError(f"request {handle}: tokens {start}..{start + n - 1} fall on pages already given back")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def group_of_run(self, run: int) -> Optional[int]:
        return self._group_of_run[run]

    def run_view(self, run: int, block_tables: Sequence[Optional[torch.Tensor]],
                 slot_mappings: Sequence[Optional[torch.Tensor]]) -> RunCacheView:
        """The view run ``run`` gets for one step, given the step's uploaded per-group tensors."""
        gi = self._group_of_run[run]
        state = self.state[run]
        if gi is None:
            return RunCacheView(None, None, None, None, self.page_size, False, state)
        g = self.groups[gi]
        owner = self._owner_of_run[run]
        i = g.run_index[owner]
        return RunCacheView(g.k_pages[i], g.v_pages[i], block_tables[gi], slot_mappings[gi],
                            self.page_size, owner == run, state, g.need.window)

    # --------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, held twice or freed twice; tables agree with the lists."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for req in self._requests.values():
                blocks = req.blocks[gi]
                want = -(-req.length // self.page_size)
                if len(blocks) != want:
                    raise AssertionError(
                        f"group {gi} request {req.handle}: {len(blocks)} blocks for {req.length} tokens")
                for b, p in enumerate(blocks):
                    if p == FREED:
                        if g.need.kind != "window" or b >= req.first_block[gi]:
                            raise AssertionError(f"group {gi} request {req.handle}: block {b} has no page")
                        continue
                    if b < req.first_block[gi]:
                        raise AssertionError(f"group {gi} request {req.handle}: block {b} kept below the window")
                    held[p] = held.get(p, 0) + 1
                row = self._tables[gi][req.slot]
                if list(row[:len(blocks)]) != blocks or (row[len(blocks):] != FREED).any():
                    raise AssertionError(f"group {gi} request {req.handle}: host block table out of date")
            free = g.allocator.free_pages()
            free_set = set(free)
            if len(free_set) != len(free):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            if free_set & set(held):
                raise AssertionError(f"group {gi}: pages both free and held: {sorted(free_set & set(held))}")
            for p in range(g.allocator.n_pages):
                rc = g.allocator.refcount(p)
                if rc != held.get(p, 0):
                    raise AssertionError(f"group {gi}: page {p} has refcount {rc} but {held.get(p, 0)} holders")
                if (rc == 0) != (p in free_set):
                    raise AssertionError(f"group {gi}: page {p} refcount {rc} disagrees with the free list")
            if len(free) + len(held) != g.allocator.n_pages:
                raise AssertionError(f"group {gi}: {g.allocator.n_pages - len(free) - len(held)} pages lost")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a slot is held twice or both free and held")
        if len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise AssertionError("a slot was lost")
        for gi in range(len(self.groups)):
            for s in self._free_slots:
                if (self._tables[gi][s] != FREED).any():
                    raise AssertionError(f"group {gi}: free slot {s} still has a block table")
