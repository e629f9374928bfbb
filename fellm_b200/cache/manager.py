"""The cache manager: pages of keys and values with a block table per request, in groups of
layers with the same need, and slots for per-request state of fixed size.

FeLLM's KV fabric keeps 16-token pages of one layer in one arena, a page list per sequence and
layer, refcounts, and a LIFO free list (crates/fellm-runtime/src/kv_fabric/storage.rs:46-59,
199-233; fabric.rs:263-305,394-459,724-736; types.rs:101-111 names group kinds FullAttention /
SlidingWindow / Recurrent); its per-request conv history is a host buffer copied into and out of
a packed batch every step (crates/fellm-runtime/src/hybrid_state.rs:63-134;
engine.rs:2813-2844,2963-2990).

Here:
  * A *group* is the set of schedule entries whose mixers declare the same need.  A PagedKV group
    owns one device pool [page][layer in group][k/v][kv head][token in page][head_dim] and one
    free list; a page holds `page_tokens` positions of ALL the group's layers, so a request has
    one block table per group.  A FixedState group owns [slot][layer in group][*shape] float32.
  * A request holds one *slot* (its row in every group's block table and state array) from
    admission to release.  State is zeroed when the slot is taken.
  * reserve() covers the positions a step is about to write, for all groups or for none;
    advance() records them as written and, for windowed groups, gives back the pages no later
    query can reach; release() gives everything back.  Freed pages go on top of the free list and
    are the next to be used.
  * Block tables live on the device ([slot][logical page] int32, -1 = no page) and are patched
    from a host mirror: only rows that changed since the last step are copied.

The accounting (PageAllocator, SlotAllocator) is plain Python and is tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config.errors import CacheError
from ..parts.base import FixedState, PagedKV


class PageAllocator:
    """Free list of page ids, LIFO.  Refuses double frees and frees of pages it never gave."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages - 1, -1, -1))      # page 0 is handed out first
        self._held = [False] * self.n_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheError("out of cache pages")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int):
        if not 0 <= page < self.n_pages or not self._held[page]:
            raise CacheError(f"page {page} freed but not held")
        self._held[page] = False
        self._free.append(page)

    def held(self) -> List[int]:
        return [p for p, h in enumerate(self._held) if h]


class SlotAllocator(PageAllocator):
    """Same discipline for request slots."""

    def alloc(self) -> int:
        if not self._free:
            raise CacheError("out of request slots")
        return super().alloc()


@dataclass
class PagedView:
    """What an attention mixer sees of its cache."""
    pool: torch.Tensor            # [pages, layers, 2, G, page_tokens, hd]
    block_table: torch.Tensor     # [slots, width] int32 on the device
    layer: int                    # index in the group
    page_tokens: int
    window: Optional[int]


@dataclass
class StateView:
    """What a mixer with fixed-size state sees: states[slot] is its state of that request."""
    states: torch.Tensor          # [slots, *shape] float32 view (slot stride covers the group)
    item_slot: Optional[torch.Tensor] = None     # [n_items] int32, set per step


class _PagedGroup:
    def __init__(self, need: PagedKV, entries, n_pages, n_slots, width, page_tokens, dtype, device):
        self.need, self.entries = need, list(entries)
        self.page_tokens, self.width = page_tokens, width
        self.alloc = PageAllocator(n_pages)
        # one page and one block-table row beyond what the allocators hand out: the padding rows of a decode
        # step (CacheManager.pad_slot) keep their single position there
        self.pool = torch.zeros((n_pages + 1, len(self.entries), 2, need.kv_heads, page_tokens,
                                 need.head_dim), dtype=dtype, device=device)
        # pageable on purpose: a copy from pageable memory is staged by the driver before the call
        # returns, so later edits of the mirror cannot reach a copy that is still queued
        self.table_host = torch.full((n_slots + 1, width), -1, dtype=torch.int32)
        self.table_dev = torch.full((n_slots + 1, width), -1, dtype=torch.int32, device=device)
        self.table_host[n_slots, 0] = n_pages
        self.table_dev[n_slots, 0] = n_pages
        self.dirty: Dict[int, List[int]] = {}            # slot -> [lo, hi) of changed entries
        self.first_page: Dict[int, int] = {}             # slot -> first logical page still held
        self.n_logical: Dict[int, int] = {}              # slot -> logical pages ever mapped

    def bytes_per_token(self) -> int:
        return len(self.entries) * 2 * self.need.kv_heads * self.need.head_dim * self.pool.element_size()

    def _mark(self, slot, lo, hi):
        d = self.dirty.get(slot)
        if d is None:
            self.dirty[slot] = [lo, hi]
        else:
            d[0], d[1] = min(d[0], lo), max(d[1], hi)

    def pages_needed(self, slot, new_len) -> int:
        want = -(-new_len // self.page_tokens)
        return max(0, want - self.n_logical.get(slot, 0))

    def grow(self, slot, new_len):
        have = self.n_logical.get(slot, 0)
        want = -(-new_len // self.page_tokens)
        if want > self.width:
            raise CacheError(f"a request of {new_len} tokens exceeds the block table "
                             f"({self.width} pages of {self.page_tokens})")
        for i in range(have, want):
            self.table_host[slot, i] = self.alloc.alloc()
        if want > have:
            self._mark(slot, have, want)
            self.n_logical[slot] = want
            self.first_page.setdefault(slot, 0)

    def trim_window(self, slot, length):
        """After `length` positions are written: pages that end at or before length-window+1
        can no longer be read."""
        if self.need.window is None or slot not in self.n_logical:
            return
        dead = max(0, length - self.need.window + 1) // self.page_tokens
        first = self.first_page.get(slot, 0)
        for i in range(first, min(dead, self.n_logical[slot])):
            self.alloc.free(int(self.table_host[slot, i]))
            self.table_host[slot, i] = -1
        if dead > first:
            self._mark(slot, first, min(dead, self.n_logical[slot]))
            self.first_page[slot] = min(dead, self.n_logical[slot])

    def release(self, slot):
        n = self.n_logical.pop(slot, 0)
        first = self.first_page.pop(slot, 0)
        for i in range(first, n):
            self.alloc.free(int(self.table_host[slot, i]))
        if n:
            self.table_host[slot, :n] = -1
            self._mark(slot, 0, n)

    def held_pages(self, slot) -> List[int]:
        n, first = self.n_logical.get(slot, 0), self.first_page.get(slot, 0)
        return [int(self.table_host[slot, i]) for i in range(first, n)]

    def flush(self):
        for slot, (lo, hi) in self.dirty.items():
            self.table_dev[slot, lo:hi].copy_(self.table_host[slot, lo:hi], non_blocking=True)
        self.dirty.clear()


class _StateGroup:
    def __init__(self, need: FixedState, entries, n_slots, device):
        self.need, self.entries = need, list(entries)
        self.states = torch.zeros((n_slots + 1, len(self.entries), *need.shape), dtype=torch.float32,
                                  device=device)               # (the last row: CacheManager.pad_slot)

    def bytes_per_request(self) -> int:
        return self.states[0].numel() * 4


class CacheManager:
    def __init__(self, needs, *, page_tokens: int, max_tokens: int, max_requests: int, n_ctx: int,
                 dtype: torch.dtype, device):
        """needs[n]: the cache need of schedule entry n: PagedKV, FixedState, None, or a list of
        them for a mixer that keeps several things (pages and a state; two states of different
        shapes, as FeLLM's GatedDeltaNet keeps a convolution history and a matrix,
        crates/fellm-model/src/graph.rs:792-806).  An entry's view is then a list in the same order.
        max_tokens: positions the page pool of each group holds (rounded up to whole pages)."""
        self.page_tokens, self.n_slots, self.n_ctx = int(page_tokens), int(max_requests), int(n_ctx)
        self.device = device
        # A slot no request ever gets, with one position of cache (a page of its own in every paged group) and
        # a state row: a step may carry rows that belong to nobody (a decode step filled up to a row count whose
        # CUDA graph exists); they read and write there and their results are dropped.
        self.pad_slot = self.n_slots
        self.slots = SlotAllocator(self.n_slots)
        self.paged: List[_PagedGroup] = []
        self.fixed: List[_StateGroup] = []
        self._entry_view: Dict[int, object] = {}
        n_pages = -(-int(max_tokens) // self.page_tokens)
        width = -(-self.n_ctx // self.page_tokens)
        by_need: Dict[object, List[tuple]] = {}          # need -> [(entry, index among the entry's needs)]
        for n, need in enumerate(needs):
            for k, one in enumerate(need if isinstance(need, (list, tuple)) else [need]):
                if one is None:
                    continue
                if not isinstance(one, (PagedKV, FixedState)):
                    raise CacheError(f"schedule entry {n}: unknown cache need {one!r}")
                by_need.setdefault(one, []).append((n, k))
        placed: Dict[tuple, object] = {}
        for need, users in by_need.items():
            if isinstance(need, PagedKV):
                g = _PagedGroup(need, users, n_pages, self.n_slots, width, self.page_tokens, dtype, device)
                self.paged.append(g)
                for li, user in enumerate(users):
                    placed[user] = PagedView(g.pool, g.table_dev, li, self.page_tokens, need.window)
            else:
                g = _StateGroup(need, users, self.n_slots, device)
                self.fixed.append(g)
                for li, user in enumerate(users):
                    placed[user] = StateView(g.states[:, li])
        for n, need in enumerate(needs):
            if isinstance(need, (list, tuple)):
                self._entry_view[n] = [placed.get((n, k)) for k in range(len(need))]
            elif need is not None:
                self._entry_view[n] = placed[(n, 0)]
        self.n_entries = len(needs)
        self._views_key, self._views = None, None
        self.has_windows = any(g.need.window is not None for g in self.paged)
        self.req_slot: Dict[object, int] = {}
        self.req_len: Dict[object, int] = {}

    # ---- sizes
    @property
    def n_pages(self) -> int:
        return min((g.alloc.n_pages for g in self.paged), default=0)

    def free_pages(self) -> int:
        return min((g.alloc.free_count for g in self.paged), default=1 << 30)

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.paged)

    @staticmethod
    def tokens_for_budget(needs, element_size: int, budget: int, page_tokens: int, cap: int) -> int:
        """Positions a pool of `budget` bytes holds, every paged group getting the same number of
        them: FeLLM's pages = budget / page_bytes (crates/fellm-runtime/src/kv_fabric/fabric.rs:
        59-61), in whole pages, at least one and at most `cap` positions."""
        per_token = 0
        for need in needs:
            for one in (need if isinstance(need, (list, tuple)) else [need]):
                if isinstance(one, PagedKV):
                    per_token += 2 * one.kv_heads * one.head_dim * element_size
        if per_token == 0:
            return page_tokens
        tokens = max(min(budget // per_token, cap), page_tokens)
        return tokens - tokens % page_tokens

    # ---- requests
    def has(self, req) -> bool:
        return req in self.req_slot

    def length(self, req) -> int:
        return self.req_len[req]

    def slot(self, req) -> int:
        return self.req_slot[req]

    def can_admit(self) -> bool:
        return self.slots.free_count > 0

    def add_request(self, req) -> int:
        if req in self.req_slot:
            raise CacheError(f"request {req!r} is already live")
        slot = self.slots.alloc()
        self.req_slot[req], self.req_len[req] = slot, 0
        for g in self.fixed:
            g.states[slot].zero_()
        return slot

    def pages_needed(self, req, n_new: int) -> int:
        """Pages (of the neediest group) that covering n_new more positions takes."""
        slot, new_len = self.req_slot[req], self.req_len[req] + n_new
        return max((g.pages_needed(slot, new_len) for g in self.paged), default=0)

    def can_reserve(self, asks) -> bool:
        """asks: [(req, n_new)] of one step, all together."""
        for g in self.paged:
            need = sum(g.pages_needed(self.req_slot[r], self.req_len[r] + n) for r, n in asks)
            if need > g.alloc.free_count:
                return False
        return True

    def reserve(self, req, n_new: int):
        """Maps pages for positions [len, len+n_new) in every paged group, or in none."""
        if req not in self.req_slot:
            raise CacheError(f"unknown request {req!r}")
        slot, new_len = self.req_slot[req], self.req_len[req] + n_new
        if new_len > self.n_ctx:
            raise CacheError(f"request {req!r} would reach {new_len} tokens; the context holds {self.n_ctx}")
        for g in self.paged:
            if g.pages_needed(slot, new_len) > g.alloc.free_count:
                raise CacheError(f"out of cache pages: request {req!r} needs {g.pages_needed(slot, new_len)}, "
                                 f"{g.alloc.free_count} free")
        for g in self.paged:
            g.grow(slot, new_len)

    def advance(self, req, n_new: int):
        """The step wrote n_new positions of `req`."""
        self.req_len[req] += n_new
        for g in self.paged:
            g.trim_window(self.req_slot[req], self.req_len[req])

    def release(self, req):
        if req not in self.req_slot:
            raise CacheError(f"request {req!r} released but not live")
        slot = self.req_slot.pop(req)
        del self.req_len[req]
        for g in self.paged:
            g.release(slot)
        self.slots.free(slot)

    def live_requests(self):
        return list(self.req_slot)

    # ---- per step
    def flush(self):
        """Copies changed block-table rows to the device (before the step's kernels)."""
        for g in self.paged:
            g.flush()

    def views(self, item_slot: Optional[torch.Tensor]):
        """Cache views per schedule entry for one step (None where an entry keeps nothing)."""
        key = None if item_slot is None else (item_slot.data_ptr(), item_slot.numel())
        if key is not None and self._views_key == key:
            return self._views
        out = []
        def of_step(v):
            return StateView(v.states, item_slot) if isinstance(v, StateView) else v
        for n in range(self.n_entries):
            v = self._entry_view.get(n)
            out.append([of_step(one) for one in v] if isinstance(v, list) else of_step(v))
        if key is not None:
            self._views_key, self._views = key, out
        return out

    # ---- checks used by tests
    def audit(self):
        """Raises CacheError when a page is held twice, lost, or free and held at once."""
        for gi, g in enumerate(self.paged):
            seen = {}
            for req, slot in self.req_slot.items():
                for p in g.held_pages(slot):
                    if p < 0:
                        raise CacheError(f"group {gi}: request {req!r} maps a freed page")
                    if p in seen:
                        raise CacheError(f"group {gi}: page {p} held by {seen[p]!r} and {req!r}")
                    seen[p] = req
            held = set(g.alloc.held())
            if held != set(seen):
                raise CacheError(f"group {gi}: allocator holds {sorted(held)}, requests map {sorted(seen)}")
            if len(held) + g.alloc.free_count != g.alloc.n_pages:
                raise CacheError(f"group {gi}: {len(held)} held + {g.alloc.free_count} free != {g.alloc.n_pages}")
            if len(set(g.alloc._free)) != len(g.alloc._free):
                raise CacheError(f"group {gi}: a page is on the free list twice")
        if len(self.req_slot) + self.slots.free_count != self.n_slots:
            raise CacheError("slots lost")
        if len(set(self.req_slot.values())) != len(self.req_slot):
            raise CacheError("a slot is held twice")
