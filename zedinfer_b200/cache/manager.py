"""The cache manager: pages of keys and values per group of layers, block tables per request,
and slots for fixed-size per-request state.

Each call of the model's schedule that owns a cache declares what it needs
(:class:`PagedKVNeed`, :class:`StateNeed` or nothing).  Calls with the same page shape and
the same window form a *group*: one pool of pages, one block table per request.  A page id
means the same page in every call of its group, so a request's table is one row per group
however many layers there are (the reference keeps one table per layer,
include/backend/kvcache/block_pool.hpp:73-103).  Groups with a window give pages back as soon
as the window has passed them; everything is given back when a request is closed.

Device layout of a group: ``[num_pages + 1, calls, 2 (k|v), kv_heads, page_size, head_dim]``.
The extra last page is a scratch page that is never handed out: padding tokens of a
captured decode step write there.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .pool import OutOfPages, PagePool, StateSlotPool


@dataclass(frozen=True)
class PagedKVNeed:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None        # None: all keys; else the last `window` keys


@dataclass(frozen=True)
class StateNeed:
    shape: Tuple[int, ...]              # per request
    dtype: torch.dtype = torch.float32


@dataclass
class CallCacheView:
    """What one call of the schedule sees of the cache."""
    kind: str                           # "paged", "state" or "none"
    group: int = -1                     # paged: index of the group (selects the block table)
    tensor: Optional[torch.Tensor] = None   # paged: this call's slice of the pool; state: [slots, *shape]
    page_stride: int = 0                # elements between pages
    kv_stride: int = 0                  # elements between the k and the v half of a page
    page_size: int = 0
    window: Optional[int] = None


@dataclass
class PagedGroup:
    n_kv_heads: int
    head_dim: int
    window: Optional[int]
    calls: List[int] = field(default_factory=list)
    pool: Optional[PagePool] = None
    tensor: Optional[torch.Tensor] = None
    num_pages: int = 0                  # pages of this group's pool; page ``num_pages`` of the tensor is the scratch page

    def page_elems(self, page_size: int) -> int:
        return len(self.calls) * 2 * self.n_kv_heads * page_size * self.head_dim


class RequestCache:
    """What one live request holds: its committed length, a block table per group, a state slot."""
    __slots__ = ("request_id", "length", "tables", "slot", "closed", "version", "serial")
    _serials = itertools.count(1)

    def __init__(self, request_id, n_groups: int, slot: int):
        self.request_id = request_id
        self.serial = next(RequestCache._serials)   # never comes back in this process, unlike a request id that is reopened
        self.length = 0
        self.version = 0                      # bumped whenever a block table changes (pages added or given back)
        self.tables: List[List[int]] = [[] for _ in range(n_groups)]
        self.slot = slot
        self.closed = False

    def pages_held(self) -> int:
        return sum(1 for t in self.tables for p in t if p >= 0)


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[int, object]], page_size: int, *, max_requests: int = 64,
                 max_step_tokens: Optional[int] = None):
        """``needs``: (cache key, need) for every cache: the schedule index of the call that owns it, or any other
        hashable key (a layer with a second mixer uses (index, role))."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        # The most tokens one step adds to one request, if the caller binds itself to that (a scheduler's token
        # budget).  A group with a window then never holds more than ``window + max_step_tokens`` tokens of a request
        # (what a step adds is only given back when the step commits), so its pool can be smaller than the others'.
        self.max_step_tokens = max_step_tokens
        self.groups: List[PagedGroup] = []
        self._call_group: Dict[object, Tuple[int, int]] = {}
        self._state_needs: Dict[object, StateNeed] = {}
        self._state_tensors: Dict[object, torch.Tensor] = {}
        for call, need in needs:
            if need is None:
                continue
            if isinstance(need, PagedKVNeed):
                for gi, g in enumerate(self.groups):
                    if (g.n_kv_heads, g.head_dim, g.window) == (need.n_kv_heads, need.head_dim, need.window):
                        break
                else:
                    gi = len(self.groups)
                    self.groups.append(PagedGroup(need.n_kv_heads, need.head_dim, need.window))
                self._call_group[call] = (gi, len(self.groups[gi].calls))
                self.groups[gi].calls.append(call)
            elif isinstance(need, StateNeed):
                self._state_needs[call] = need
            else:
                raise TypeError(f"call {call}: unknown cache need {need!r}")
        self.slots = StateSlotPool(max_requests if self._state_needs else 0)
        self.max_requests = max_requests
        self._requests: Dict[object, RequestCache] = {}
        self.device: Optional[torch.device] = None
        self.dtype: Optional[torch.dtype] = None

    # ---- sizing ---------------------------------------------------------------------------
    def bytes_per_page_all_groups(self, dtype: torch.dtype) -> int:
        item = torch.empty((), dtype=dtype).element_size()
        return sum(g.page_elems(self.page_size) for g in self.groups) * item

    def state_bytes(self) -> int:
        total = 0
        for need in self._state_needs.values():
            n = 1
            for s in need.shape:
                n *= s
            total += n * torch.empty((), dtype=need.dtype).element_size() * self.max_requests
        return total

    def group_pages(self, g: PagedGroup, num_pages: int) -> int:
        """Pages of group ``g`` when the groups that keep all keys get ``num_pages``: as many, or, for a group with a
        window under a bound on a step's tokens, what ``max_requests`` requests can hold at most."""
        if g.window is None or self.max_step_tokens is None:
            return num_pages
        # window - 1 + step tokens, starting anywhere in a page
        per_request = (g.window + self.max_step_tokens + self.page_size - 2) // self.page_size + 1
        return max(1, min(num_pages, per_request * self.max_requests))

    def pool_bytes(self, num_pages: int, dtype: torch.dtype) -> int:
        item = torch.empty((), dtype=dtype).element_size()
        return sum(g.page_elems(self.page_size) * (self.group_pages(g, num_pages) + 1) for g in self.groups) * item

    def pages_for_budget(self, budget_bytes: int, dtype: torch.dtype) -> int:
        """The largest page count of the groups without a window (each group has one scratch page more) whose pools
        and state fit in ``budget_bytes``."""
        if not self.groups:
            return 1
        budget = budget_bytes - self.state_bytes()
        lo, hi = 0, 1
        while self.pool_bytes(hi, dtype) <= budget and hi < (1 << 40):
            lo, hi = hi, hi * 2
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self.pool_bytes(mid, dtype) <= budget:
                lo = mid
            else:
                hi = mid
        return lo

    def set_num_pages(self, num_pages: int) -> None:
        """Host bookkeeping only (tests of the manager and the scheduler need no device)."""
        if num_pages <= 0:
            raise ValueError(f"the cache needs at least one page per group, got {num_pages}")
        if self._requests:
            raise RuntimeError("cannot resize the cache while requests are live")
        for g in self.groups:
            g.num_pages = self.group_pages(g, num_pages)
            g.pool = PagePool(g.num_pages)
        self.num_pages = num_pages

    def allocate_device(self, num_pages: int, dtype: torch.dtype, device) -> None:
        self.set_num_pages(num_pages)
        self.device, self.dtype = torch.device(device), dtype
        for g in self.groups:
            # zeroed: attention multiplies slots that hold nothing yet by probability 0, which must not meet NaN bits
            g.tensor = torch.zeros((g.num_pages + 1, len(g.calls), 2, g.n_kv_heads, self.page_size, g.head_dim),
                                   dtype=dtype, device=device)
        for call, need in self._state_needs.items():
            self._state_tensors[call] = torch.zeros((self.max_requests,) + tuple(need.shape), dtype=need.dtype,
                                                    device=device)

    @property
    def step_bound(self) -> Optional[int]:
        """The most tokens of one request that a step may bring, where the pools rely on it (some group has a window
        and the caller gave ``max_step_tokens``); None where nothing depends on it."""
        if self.max_step_tokens is not None and any(g.window is not None for g in self.groups):
            return self.max_step_tokens
        return None

    @property
    def scratch_pages(self) -> List[int]:
        """Per group, the page behind the pool's last: padding rows write there, and block-table entries whose page
        a window has given back point there."""
        return [g.num_pages for g in self.groups]

    def view_for_call(self, call) -> CallCacheView:
        if call in self._call_group:
            gi, j = self._call_group[call]
            g = self.groups[gi]
            t = g.tensor[:, j] if g.tensor is not None else None
            return CallCacheView("paged", gi, t,
                                 page_stride=g.page_elems(self.page_size),
                                 kv_stride=g.n_kv_heads * self.page_size * g.head_dim,
                                 page_size=self.page_size, window=g.window)
        if call in self._state_needs:
            return CallCacheView("state", tensor=self._state_tensors.get(call))
        return CallCacheView("none")

    # ---- requests -------------------------------------------------------------------------
    @property
    def num_live(self) -> int:
        return len(self._requests)

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def min_free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=1 << 30)

    def open(self, request_id) -> RequestCache:
        if request_id in self._requests:
            raise ValueError(f"request {request_id!r} is already live")
        if self.step_bound is not None and len(self._requests) >= self.max_requests:
            raise RuntimeError(f"{self.max_requests} requests are live already: the pools of the groups with a window "
                               "are sized for that many")
        slot = -1
        if self.slots.num_slots:
            slot = self.slots.acquire_slot()
            for t in self._state_tensors.values():
                t[slot].zero_()
        rc = RequestCache(request_id, len(self.groups), slot)
        self._requests[request_id] = rc
        return rc

    def reset_state(self, rc: RequestCache) -> None:
        """Zero the fixed-size state of ``rc`` in every call that keeps one (a request that starts over, e.g. after
        preemption with the same slot); the reference's ``reset_slot`` (include/frontend/models/ssm_state_pool.hpp:61-131)."""
        if rc.slot >= 0:
            for t in self._state_tensors.values():
                t[rc.slot].zero_()

    def copy_state(self, src: RequestCache, dst: RequestCache) -> None:
        """``dst``'s fixed-size state := ``src``'s, in every call that keeps one (a request that continues from
        another's state); the reference's ``copy_slot_state``."""
        if src.slot < 0 or dst.slot < 0:
            raise ValueError("copy_state needs two requests that hold state slots")
        for t in self._state_tensors.values():
            t[dst.slot].copy_(t[src.slot])

    def get(self, request_id) -> Optional[RequestCache]:
        return self._requests.get(request_id)

    def can_open(self) -> bool:
        return self.slots.num_slots == 0 or self.slots.num_free_slots > 0

    def _first_needed_block(self, g: PagedGroup, length: int) -> int:
        """Index of the first block a request of ``length`` committed tokens still needs."""
        if g.window is None:
            return 0
        first_token = max(0, length - g.window + 1)      # the next query (position >= length) reads from here
        return first_token // self.page_size

    def pages_needed(self, rc: Optional[RequestCache], new_len: int) -> List[int]:
        """Pages per group that ``ensure(rc, new_len)`` would take (``rc=None``: a fresh request).  A group with a
        window under a bound on a step's tokens takes pages only as far as the next step can reach: what lies
        further ahead (a whole prompt reserved at admission) it will take step by step, as the window gives the
        pages behind it back, and its pool is sized so that this cannot fail."""
        length = rc.length if rc is not None else 0
        out = []
        for gi, g in enumerate(self.groups):
            reach = new_len
            if g.window is not None and self.max_step_tokens is not None:
                reach = min(new_len, length + self.max_step_tokens)
            want = (reach + self.page_size - 1) // self.page_size
            have = len(rc.tables[gi]) if rc is not None else 0
            out.append(max(0, want - have))
        return out

    def can_ensure(self, rc: Optional[RequestCache], new_len: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(rc, new_len), self.groups))

    def ensure(self, rc: RequestCache, new_len: int) -> None:
        """Give ``rc`` pages for tokens ``[rc.length, new_len)`` in every group, or change nothing and raise."""
        if rc.closed:
            raise RuntimeError(f"request {rc.request_id!r} is closed")
        if all(new_len <= len(t) * self.page_size for t in rc.tables):
            return                              # the pages are there already (the usual case of a decode step)
        needed = self.pages_needed(rc, new_len)
        for n, g in zip(needed, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {rc.request_id!r} needs {n} more pages for {new_len} tokens, "
                                 f"{g.pool.num_free} free")
        for gi, (n, g) in enumerate(zip(needed, self.groups)):
            if n:
                rc.tables[gi].extend(g.pool.allocate_many(n))
                rc.version += 1

    def commit(self, rc: RequestCache, new_len: int) -> None:
        """The step that wrote tokens up to ``new_len`` is done: advance, release what a window has passed."""
        if new_len < rc.length:
            raise ValueError("a request's length cannot shrink")
        rc.length = new_len
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            table = rc.tables[gi]
            for b in range(min(self._first_needed_block(g, new_len), len(table))):
                if table[b] >= 0:
                    g.pool.free(table[b])
                    table[b] = -1
                    rc.version += 1

    def close(self, rc: RequestCache) -> None:
        if rc.closed:
            raise ValueError(f"request {rc.request_id!r} is closed twice")
        for gi, g in enumerate(self.groups):
            for p in rc.tables[gi]:
                if p >= 0:
                    g.pool.free(p)
            rc.tables[gi] = []
        if rc.slot >= 0:
            self.slots.release_slot(rc.slot)
            rc.slot = -1
        rc.closed = True
        del self._requests[rc.request_id]

    def check(self) -> None:
        """No page lost, held twice or freed twice; every held page belongs to exactly one live request."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            owned: Dict[int, object] = {}
            for rc in self._requests.values():
                for p in rc.tables[gi]:
                    if p < 0:
                        continue
                    if p in owned:
                        raise AssertionError(f"group {gi}: page {p} is held by {owned[p]!r} and {rc.request_id!r}")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"group {gi}: page {p} of {rc.request_id!r} is on the free list")
                    owned[p] = rc.request_id
            if len(owned) != g.pool.num_used:
                raise AssertionError(f"group {gi}: {g.pool.num_used} pages held, {len(owned)} owned by requests")
        self.slots.check()
