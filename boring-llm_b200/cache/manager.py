"""The cache manager: keys and values in fixed-size pages with a block table for each request,
one pool per group of layers with the same needs, and slots for per-request state of fixed size.

The reference keeps one contiguous, grown-by-copy buffer per layer (main + tail of up to 63 rows,
src/model.br:1670-1695) for its single sequence, truncates by setting a length (:2313-2314) and
treats windows as masks over the full cache (README.md:237). Pages, block tables, groups and
slots are this engine's own design in the role of src/kvplane.br; what carries over is that a
cache is only ever read up to the request's length, so freed pages need no clearing.

Everything here is host-side bookkeeping and runs without a GPU; `storage.CacheStorage` owns the
device tensors that the page and slot numbers index.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union


@dataclass(frozen=True)
class PagedKVSpec:
    """What a mixer that caches keys and values needs: `window` 0 keeps every key, n > 0 only the
    last n positions (the query's own included)."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (a recurrent state, a running sum): one tensor of `shape`
    per request and cache layer, zero when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"


CacheSpec = Union[PagedKVSpec, StateSpec, None]


class CacheError(RuntimeError):
    """A misuse of the manager (unknown request, double free, ...): a bug of the caller."""


class PagePool:
    """Free pages of one group, handed out last-freed-first so that small pools reuse pages at once."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._owner: List[Optional[object]] = [None] * num_pages
        self.high_water = 0
        self.freed_log: Optional[List[int]] = None     # when a list: every page given back is noted here (debugging)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, owner) -> int:
        if not self._free:
            raise CacheError("page pool is empty (reserve() must check before taking)")
        p = self._free.pop()
        if self._owner[p] is not None:
            raise CacheError(f"page {p} was on the free list while owned by {self._owner[p]!r}")
        self._owner[p] = owner
        self.high_water = max(self.high_water, self.num_pages - len(self._free))
        return p

    def give_back(self, page: int, owner) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool")
        if self._owner[page] is None:
            raise CacheError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise CacheError(f"page {page} is owned by {self._owner[page]!r}, not by {owner!r}")
        self._owner[page] = None
        self._free.append(page)
        if self.freed_log is not None:
            self.freed_log.append(page)

    def owner_of(self, page: int):
        return self._owner[page]


@dataclass
class PagedGroup:
    spec: PagedKVSpec
    cache_layers: List[int]          # cache ids that share this group's block tables
    pool: PagePool


@dataclass
class StateGroup:
    spec: StateSpec
    cache_layers: List[int]


@dataclass
class RequestCache:
    """What one live request holds: a slot, its length, and one block table per paged group.
    A table entry of -1 is a page that a window has passed and that was given back."""
    request_id: object
    slot: int
    num_tokens: int = 0
    tables: List[List[int]] = field(default_factory=list)
    uid: int = 0          # unlike request_id never used twice by one manager
    version: int = 0      # counts the changes of `tables`: (uid, version) names one state of the block tables


class CacheManager:
    def __init__(self, specs: Sequence[CacheSpec], page_size: int, capacity_tokens: int,
                 max_requests: int, on_slot_assigned: Optional[Callable[[int], None]] = None):
        """`specs[c]` is what cache layer `c` needs (None: nothing). Layers with equal needs form
        a group; every paged group gets a pool of ceil(capacity_tokens / page_size) pages."""
        if page_size <= 0 or capacity_tokens <= 0 or max_requests <= 0:
            raise ValueError("page_size, capacity_tokens and max_requests must be positive")
        self.page_size = page_size
        self.capacity_tokens = capacity_tokens
        self.max_requests = max_requests
        self.num_pages = -(-capacity_tokens // page_size)
        self.paged_groups: List[PagedGroup] = []
        self.state_groups: List[StateGroup] = []
        # cache layer -> ("paged" | "state", group index, index inside the group)
        self.layer_location: Dict[int, Tuple[str, int, int]] = {}
        for c, spec in enumerate(specs):
            if spec is None:
                continue
            if isinstance(spec, PagedKVSpec):
                if spec.window < 0:
                    raise ValueError(f"cache layer {c}: window must not be negative")
                for gi, g in enumerate(self.paged_groups):
                    if g.spec == spec:
                        break
                else:
                    gi = len(self.paged_groups)
                    self.paged_groups.append(PagedGroup(spec, [], PagePool(self.num_pages)))
                g = self.paged_groups[gi]
                self.layer_location[c] = ("paged", gi, len(g.cache_layers))
                g.cache_layers.append(c)
            elif isinstance(spec, StateSpec):
                for gi, sg in enumerate(self.state_groups):
                    if sg.spec == spec:
                        break
                else:
                    gi = len(self.state_groups)
                    self.state_groups.append(StateGroup(spec, []))
                sg = self.state_groups[gi]
                self.layer_location[c] = ("state", gi, len(sg.cache_layers))
                sg.cache_layers.append(c)
            else:
                raise TypeError(f"cache layer {c}: unknown cache spec {spec!r}")
        self._free_slots: List[int] = list(range(max_requests - 1, -1, -1))
        self._requests: Dict[object, RequestCache] = {}
        self._on_slot_assigned = on_slot_assigned
        self._next_uid = 0

    # ---- requests -------------------------------------------------------------------------
    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def add_request(self, request_id) -> RequestCache:
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise CacheError("no free request slot (check has_free_slot() before admitting)")
        slot = self._free_slots.pop()
        rc = RequestCache(request_id, slot, 0, [[] for _ in self.paged_groups], self._next_uid)
        self._next_uid += 1
        self._requests[request_id] = rc
        if self._on_slot_assigned is not None:
            self._on_slot_assigned(slot)       # the storage zeroes the slot's state
        return rc

    def get(self, request_id) -> RequestCache:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def find(self, request_id) -> Optional[RequestCache]:
        """The live request's record, or None."""
        return self._requests.get(request_id)

    def __contains__(self, request_id) -> bool:
        return request_id in self._requests

    def live_requests(self):
        return list(self._requests)

    # ---- pages ----------------------------------------------------------------------------
    def _pages_needed(self, rc: RequestCache, n_new: int) -> List[int]:
        total = -(-(rc.num_tokens + n_new) // self.page_size)
        return [max(0, total - len(t)) for t in rc.tables]

    def can_reserve(self, request_id, n_new: int) -> bool:
        rc = self.get(request_id)
        need = self._pages_needed(rc, n_new)
        return all(n <= g.pool.num_free for n, g in zip(need, self.paged_groups))

    def pages_short(self, request_id, n_new: int) -> int:
        """How many pages the fullest group lacks for `n_new` more tokens (0: it fits)."""
        rc = self.get(request_id)
        need = self._pages_needed(rc, n_new)
        return max([0] + [n - g.pool.num_free for n, g in zip(need, self.paged_groups)])

    def reserve(self, request_id, n_new: int) -> bool:
        """Gives the request pages for `n_new` more tokens in every group, or none at all."""
        if n_new <= 0:
            raise CacheError("reserve() needs a positive number of tokens")
        rc = self.get(request_id)
        need = self._pages_needed(rc, n_new)
        if any(n > g.pool.num_free for n, g in zip(need, self.paged_groups)):
            return False
        for n, g, table in zip(need, self.paged_groups, rc.tables):
            for _ in range(n):
                table.append(g.pool.take(request_id))
            if n:
                rc.version += 1
        return True

    def commit(self, request_id, n_new: int) -> None:
        """The step has written `n_new` tokens. Pages that every later query's window has passed
        go back to their pool: a query at position p sees keys j with j + window > p
        (src/math.br:327-328), so page i is dead once (i + 1) * page_size <= p - window + 1."""
        rc = self.get(request_id)
        rc.num_tokens += n_new
        for table in rc.tables:
            if rc.num_tokens > len(table) * self.page_size:
                raise CacheError(f"request {request_id!r}: committed past its reserved pages")
        for g, table in zip(self.paged_groups, rc.tables):
            w = g.spec.window
            if w <= 0:
                continue
            first_needed = rc.num_tokens - w + 1
            dead = min(len(table), max(0, first_needed) // self.page_size)
            for i in range(dead):
                if table[i] >= 0:
                    g.pool.give_back(table[i], request_id)
                    table[i] = -1
                    rc.version += 1

    def truncate(self, request_id, n_keep: int) -> None:
        """Keeps the first `n_keep` tokens (the reference truncates by setting a length,
        src/model.br:2313-2314). Not possible once a window has given pages of that prefix back."""
        rc = self.get(request_id)
        if not 0 <= n_keep <= rc.num_tokens:
            raise CacheError(f"truncate({n_keep}) outside 0..{rc.num_tokens}")
        keep_pages = -(-n_keep // self.page_size)
        for g, table in zip(self.paged_groups, rc.tables):
            w = g.spec.window
            if w > 0 and n_keep < rc.num_tokens:
                first_needed = max(0, n_keep - w + 1) // self.page_size
                if any(p < 0 for p in table[first_needed:keep_pages]):
                    raise CacheError("truncate: a window has already given pages of the kept prefix back")
            while len(table) > keep_pages:
                p = table.pop()
                rc.version += 1
                if p >= 0:
                    g.pool.give_back(p, request_id)
        rc.num_tokens = n_keep

    def free(self, request_id) -> None:
        """The request ends (or is preempted): every page and its slot go back."""
        rc = self.get(request_id)
        for g, table in zip(self.paged_groups, rc.tables):
            for p in reversed(table):
                if p >= 0:
                    g.pool.give_back(p, request_id)
            table.clear()
        del self._requests[request_id]
        self._free_slots.append(rc.slot)

    # ---- figures and checks ---------------------------------------------------------------
    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.paged_groups]

    def stats(self) -> dict:
        return {
            "pages_total": self.num_pages,
            "pages_in_use": [self.num_pages - g.pool.num_free for g in self.paged_groups],
            "pages_high_water": [g.pool.high_water for g in self.paged_groups],
            "live_requests": len(self._requests),
        }

    def check(self) -> None:
        """No page lost, held twice or both free and held; slots likewise. Raises CacheError."""
        for gi, g in enumerate(self.paged_groups):
            held: Dict[int, object] = {}
            for rid, rc in self._requests.items():
                for p in rc.tables[gi]:
                    if p < 0:
                        continue
                    if p in held:
                        raise CacheError(f"group {gi}: page {p} held by {held[p]!r} and {rid!r}")
                    held[p] = rid
                    if g.pool.owner_of(p) != rid:
                        raise CacheError(f"group {gi}: page {p} in {rid!r}'s table but owned by {g.pool.owner_of(p)!r}")
            free = list(g.pool._free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {gi}: a page is on the free list twice")
            if set(free) & set(held):
                raise CacheError(f"group {gi}: pages both free and held: {sorted(set(free) & set(held))}")
            if len(free) + len(held) != g.pool.num_pages:
                raise CacheError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages lost")
        slots = [rc.slot for rc in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice or both free and held")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a request slot is lost")
