"""The cache: a slot per live sequence, keys and values for every layer that
keeps them, each sequence with its own length, and fixed-size state per slot.

Storage is paged: a page holds PAGE_TOKENS tokens of one layer,
[K|V][kv_head][token][head_dim]; a slot's block table maps its logical pages to
pool pages, so the cache is sized by the tokens that live requests hold (each
request rounded up to whole pages), not by slots times the longest sequence.

Layers with the same needs (kv heads, head size, window) form a group with
storage, block table and free list of its own.  A group with a window gives a
slot's pages back as soon as every key in them has left the window.

The reference declares per layer {kv_heads, head_dim, sliding_window, stores,
source} and keeps one contiguous buffer per storing layer for its single
sequence (src/architectures/core/kv.zig:13-38, src/runtime/session.zig:342-358);
slots, pages and groups are this library's answer to batches of sequences.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..config.spec import ScheduleEntry
from ..kernels import PAGE_TOKENS
from ..parts.base import CacheRequest, CacheView, LayerIO, StateRequest
from .pages import CacheBookkeepingError, CacheFull, FreeList


def pages_for(tokens: int) -> int:
    return (tokens + PAGE_TOKENS - 1) // PAGE_TOKENS


class TableStager:
    """Carries new block-table entries to the GPU without making the host wait.

    A copy from pageable memory blocks the host until the stream has drained, which
    would stop a decode loop that queues steps ahead every time a row crosses a page
    edge.  So the entries of one ``reserve`` are written into one of a few pinned
    buffers and copied from there in stream order; a buffer is written again only
    after the copies that read it have run (an event per buffer)."""

    RING = 4

    def __init__(self, capacity: int, device):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.capacity = max(1, int(capacity))
        self.bufs = [torch.zeros(self.capacity, dtype=torch.int32, pin_memory=self.cuda) for _ in range(self.RING)]
        self.events: List[Optional["torch.cuda.Event"]] = [None] * self.RING
        self.turn = 0
        self.fill = 0
        self.open = False

    def begin(self) -> None:
        self.turn = (self.turn + 1) % self.RING
        ev = self.events[self.turn]
        if ev is not None:
            ev.synchronize()
            self.events[self.turn] = None
        self.fill = 0
        self.open = True

    def copy(self, dst: torch.Tensor, values: Sequence[int]) -> None:
        """dst (a slice of a device table) = values."""
        k = len(values)
        if not self.open or self.fill + k > self.capacity:
            dst.copy_(torch.tensor(values, dtype=torch.int32))      # no staging room: the plain, waiting way
            return
        src = self.bufs[self.turn][self.fill:self.fill + k]
        src.numpy()[:] = values
        self.fill += k
        dst.copy_(src, non_blocking=True)

    def end(self) -> None:
        if self.open and self.fill and self.cuda:
            ev = torch.cuda.Event()
            ev.record()
            self.events[self.turn] = ev
        self.open = False


class CacheGroup:
    """Storage of the schedule entries that share one CacheRequest."""

    def __init__(self, request: CacheRequest, entries: List[int], num_pages: int, num_slots: int,
                 max_pages_per_slot: int, dtype: torch.dtype, device, stager: Optional[TableStager] = None):
        self.request = request
        self.stager = stager
        self.entries = entries
        self.num_pages = num_pages
        self.pages = FreeList(num_pages, "page")
        if request.token_shape is not None:
            shape = (PAGE_TOKENS, *request.token_shape)            # the mixer's own record per token
        else:
            shape = (2, request.num_kv_heads, PAGE_TOKENS, request.head_dim)
        self.pool = torch.zeros((len(entries), num_pages, *shape), dtype=request.dtype or dtype, device=device)
        self.block_table = torch.zeros((num_slots, max_pages_per_slot), dtype=torch.int32, device=device)
        # logical page -> pool page (or -1 once given back by the window) per slot
        self.slot_pages: Dict[int, List[int]] = {}

    @property
    def window(self) -> int:
        return self.request.window

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, pages_for(new_len) - len(self.slot_pages.get(slot, [])))

    def extend(self, slot: int, new_len: int) -> None:
        have = self.slot_pages.setdefault(slot, [])
        need = pages_for(new_len) - len(have)
        if need <= 0:
            return
        if pages_for(new_len) > self.block_table.shape[1]:
            raise CacheFull(f"a sequence of {new_len} tokens is longer than the cache allows "
                            f"({self.block_table.shape[1] * PAGE_TOKENS})")
        new = self.pages.take(need)
        a = len(have)
        have.extend(new)
        if self.stager is not None:
            self.stager.copy(self.block_table[slot, a:a + need], new)
        else:
            self.block_table[slot, a:a + need] = torch.tensor(new, dtype=torch.int32)

    def trim(self, slot: int, length: int) -> None:
        """Window groups: give back the pages whose keys can no longer be read.  The
        next query sits at position ``length`` and reads keys >= length + 1 - window."""
        if not self.window:
            return
        first_needed = max(0, length + 1 - self.window)
        have = self.slot_pages.get(slot, [])
        back = []
        for lp in range(min(len(have), first_needed // PAGE_TOKENS)):
            if have[lp] >= 0:
                back.append(have[lp])
                have[lp] = -1
        if back:
            self.pages.give(back)

    def release(self, slot: int) -> None:
        have = self.slot_pages.pop(slot, [])
        self.pages.give([p for p in have if p >= 0])


class KVCache:
    """Slots, groups and per-slot state for one model.

    requests / states: what each schedule entry's mixer asked for (None: nothing).
    max_tokens: tokens that live sequences may hold together, each rounded up to
    whole pages.  max_slots: sequences alive at once.  max_seq_len: longest sequence.
    """

    def __init__(self, schedule: Sequence[ScheduleEntry], requests: Sequence[Optional[CacheRequest]],
                 states: Sequence[Optional[StateRequest]], max_tokens: int, max_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device):
        self.device = device
        self.dtype = dtype
        self.num_pages = pages_for(max_tokens)
        if self.num_pages <= 0:
            raise ValueError("the cache needs room for at least one page of tokens")
        self.max_slots = int(max_slots)
        self.max_seq_len = int(max_seq_len)
        # a table row has a place for every page of the longest sequence: a window group gives
        # pages back as it goes, so its sequences may be longer than the pool
        max_pages_per_slot = pages_for(self.max_seq_len)
        self.slots = FreeList(self.max_slots, "slot")
        self.lengths: Dict[int, int] = {}

        # groups by request, over the entries that keep a cache of their own
        by_req: Dict[CacheRequest, List[int]] = {}
        for i, (e, r) in enumerate(zip(schedule, requests)):
            if r is not None and e.cache_of is None:
                by_req.setdefault(r, []).append(i)
        self.table_stager = TableStager(self.num_pages * max(1, len(by_req)), device)
        self.groups: List[CacheGroup] = [
            CacheGroup(r, ents, self.num_pages, self.max_slots, max_pages_per_slot, dtype, device,
                       self.table_stager)
            for r, ents in by_req.items()]
        where: Dict[int, Tuple[CacheGroup, int]] = {}
        for g in self.groups:
            for j, ent in enumerate(g.entries):
                where[ent] = (g, j)

        self.ios: List[LayerIO] = []
        self.state_tensors: List[torch.Tensor] = []
        for i, (e, r, s) in enumerate(zip(schedule, requests, states)):
            view = None
            if r is not None:
                src = i if e.cache_of is None else e.cache_of
                if src not in where:
                    raise ValueError(f"schedule[{i}] reads the cache of entry {src}, which keeps none")
                g, j = where[src]
                if e.cache_of is not None and (g.request.num_kv_heads, g.request.head_dim, g.request.token_shape,
                                               g.request.dtype) != (r.num_kv_heads, r.head_dim, r.token_shape, r.dtype):
                    raise ValueError(f"schedule[{i}] cannot read the cache of entry {src}: different head layout")
                view = CacheView(pool=g.pool[j], block_table=g.block_table, writes=e.cache_of is None, group=g)
            st = None
            if s is not None:
                st = torch.zeros((self.max_slots, *s.shape), dtype=s.dtype, device=device)
                self.state_tensors.append(st)
            self.ios.append(LayerIO(cache=view, state=st))

    # ---- slots ------------------------------------------------------------------
    def alloc_slot(self) -> int:
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        for st in self.state_tensors:
            st[slot].zero_()
        return slot

    def free_slot(self, slot: int) -> None:
        if slot not in self.lengths:
            raise CacheBookkeepingError(f"slot {slot} is freed but is not held")
        for g in self.groups:
            g.release(slot)
        del self.lengths[slot]
        self.slots.give([slot])

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    # ---- growth -----------------------------------------------------------------
    def reserve(self, growth: Sequence[Tuple[int, int]]) -> None:
        """Makes room for (slot, new tokens) pairs, all or nothing: raises CacheFull
        before anything is taken if the pages do not suffice."""
        for slot, n in growth:
            if slot not in self.lengths:
                raise CacheBookkeepingError(f"slot {slot} is not held")
            if self.lengths[slot] + n > self.max_seq_len:
                raise CacheFull(f"slot {slot}: {self.lengths[slot]} + {n} tokens exceed the longest "
                                f"sequence the cache was built for ({self.max_seq_len})")
        for g in self.groups:
            need = sum(g.pages_needed(slot, self.lengths[slot] + n) for slot, n in growth)
            if need > g.pages.available:
                raise CacheFull(f"the step needs {need} more pages of {PAGE_TOKENS} tokens, "
                                f"{g.pages.available} of {g.num_pages} are free")
        self.table_stager.begin()
        try:
            for g in self.groups:
                for slot, n in growth:
                    g.extend(slot, self.lengths[slot] + n)
        finally:
            self.table_stager.end()

    def commit(self, growth: Sequence[Tuple[int, int]]) -> None:
        """After the step ran: the sequences are longer now."""
        for slot, n in growth:
            self.lengths[slot] += n
            for g in self.groups:
                g.trim(slot, self.lengths[slot])

    # ---- checks -----------------------------------------------------------------
    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pages.check()
            owned = [p for pages in g.slot_pages.values() for p in pages if p >= 0]
            if len(owned) != len(set(owned)):
                raise CacheBookkeepingError("a page belongs to two slots")
            if len(owned) != g.pages.held:
                raise CacheBookkeepingError("held pages and the slots' pages disagree")

    def tokens_held(self) -> int:
        return max((g.pages.held for g in self.groups), default=0) * PAGE_TOKENS

    def bytes_per_token(self) -> int:
        return sum(g.pool[0, 0].numel() // PAGE_TOKENS * g.pool.element_size() * len(g.entries) for g in self.groups)
