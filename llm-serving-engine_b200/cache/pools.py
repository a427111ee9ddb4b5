"""Device tensors of the cache and the grouping of cache layers by what they keep.

Keys and values of a group live in one tensor ``[layers, 2, pages, kv_heads, page_tokens,
head_dim]`` (``[layers, 1, ...]`` for a group that keeps one row per token, which is then both): the rows of one (page, head) are contiguous (``page_tokens * head_dim`` elements), so
a kernel that walks a request's context for one head reads whole contiguous runs. Fixed-size
per-request state lives in ``[layers, max_requests, *shape]`` tensors, indexed by state slot.

Every key/value tensor has one page more than the manager hands out, and every state tensor one
slot more (``spare_page(group)``, ``spare_slot``): rows that only pad a captured batch to its fixed
size write there, where no request ever reads.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import PagedKVNeed, StateNeed, flatten_needs
from .manager import KVGroupSpec, StateGroupSpec


def group_cache_layers(needs: dict[int, object], page_tokens: int):
    """Sort cache layers into key/value groups (same heads, head size, window, kept first tokens and page dtype) and
    state groups. A cache layer may need several things at once (a tuple: at most one set of
    pages, any number of states): a state group lists such a layer once per state it holds there."""
    kv: dict[tuple, list[int]] = {}
    st: dict[tuple, list[int]] = {}
    for cid in sorted(needs):
        paged = 0
        for need in flatten_needs(needs[cid]):
            if isinstance(need, PagedKVNeed):
                paged += 1
                if paged > 1:
                    raise TypeError(f"cache layer {cid}: more than one set of pages")
                kv.setdefault((need.num_kv_heads, need.head_dim, need.window, need.dtype,
                               2 if need.values else 1, need.keep_first if need.window > 0 else 0), []).append(cid)
            elif isinstance(need, StateNeed):
                st.setdefault((tuple(need.shape), need.dtype), []).append(cid)
            else:
                raise TypeError(f"cache layer {cid}: unknown need {need!r}")
    kv_groups = [
        KVGroupSpec(tuple(ids), nk, d, w, page_tokens, dt, planes, keep)
        for (nk, d, w, dt, planes, keep), ids in kv.items()
    ]
    state_groups = [StateGroupSpec(tuple(ids), shape, dt) for (shape, dt), ids in st.items()]
    return kv_groups, state_groups


def pages_for_memory(groups, mem_bytes: int, dtype_bytes: int, max_len: int, max_portion: int):
    """Split ``mem_bytes`` between the groups in proportion to what one full-length request holds."""
    weights = [g.bytes_per_token(dtype_bytes) * g.live_tokens(max_len, max_portion) for g in groups]
    total = sum(weights) or 1
    out = []
    for g, w in zip(groups, weights):
        page_bytes = g.bytes_per_token(dtype_bytes) * g.page_tokens
        out.append(max(1, int(mem_bytes * w / total) // page_bytes))
    return out


@dataclass
class CacheView:
    """What one run of a layer sees of the cache."""

    group: int  # index of the key/value group (selects the block table), -1 if none
    page_tokens: int
    k: torch.Tensor | None  # [pages, kv_heads, page_tokens, head_dim]
    v: torch.Tensor | None
    state: torch.Tensor | None  # [max_requests, *shape]: the first (often the only) state
    writes: bool
    states: tuple = ()  # every state of the cache layer, in the order its needs were declared

    def part(self, pages: bool, first_state: int, num_states: int) -> "CacheView":
        """The view of one of several parts that share the cache layer: with or without the
        pages, and ``num_states`` of the states starting at ``first_state``."""
        st = self.states[first_state : first_state + num_states]
        return CacheView(self.group if pages else -1, self.page_tokens if pages else 0,
                         self.k if pages else None, self.v if pages else None,
                         st[0] if st else None, self.writes, tuple(st))


class CachePools:
    def __init__(self, kv_groups, state_groups, num_pages, max_requests, dtype, device) -> None:
        self.kv_groups = list(kv_groups)
        self.state_groups = list(state_groups)
        self.num_pages = list(num_pages)
        self.max_requests = max_requests
        self.kv = [
            torch.zeros(
                len(g.cache_ids), g.planes, n + 1, g.num_kv_heads, g.page_tokens, g.head_dim,
                dtype=g.dtype or dtype, device=device,
            )
            for g, n in zip(self.kv_groups, self.num_pages)
        ]
        self.state = [
            torch.zeros(len(g.cache_ids), max_requests + 1, *g.shape, dtype=g.dtype, device=device)
            for g in self.state_groups
        ]
        self._pages_of: dict[int, tuple[int, int]] = {}
        for gi, g in enumerate(self.kv_groups):
            for li, cid in enumerate(g.cache_ids):
                self._pages_of[cid] = (gi, li)
        self._states_of: dict[int, list[tuple[int, int]]] = {}
        for gi, g in enumerate(self.state_groups):
            for li, cid in enumerate(g.cache_ids):
                self._states_of.setdefault(cid, []).append((gi, li))
        self._order: dict[int, list[tuple[tuple, object]]] = {}
        self._state_views: dict[int, tuple] = {}

    def declare_order(self, needs: dict[int, object]) -> None:
        """Remember in which order each cache layer declared its states, so that ``view().states``
        follows it (states of equal shape keep their order within their group anyway)."""
        self._state_views.clear()
        for cid, need in needs.items():
            self._order[cid] = [(tuple(n.shape), n.dtype) for n in flatten_needs(need)
                                if isinstance(n, StateNeed)]

    def _states(self, cache_id: int) -> tuple:
        got = self._state_views.get(cache_id)
        if got is None:
            held = list(self._states_of.get(cache_id, ()))
            states = []
            for key in self._order.get(cache_id, ()):  # declared order
                for i, (gi, li) in enumerate(held):
                    g = self.state_groups[gi]
                    if (tuple(g.shape), g.dtype) == key:
                        states.append(self.state[gi][li])
                        del held[i]
                        break
            states += [self.state[gi][li] for gi, li in held]
            got = self._state_views[cache_id] = tuple(states)
        return got

    def view(self, cache_id: int, writes: bool) -> CacheView:
        where = self._pages_of.get(cache_id)
        states = self._states(cache_id)
        first = states[0] if states else None
        if where is None:
            return CacheView(-1, 0, None, None, first, writes, states)
        gi, li = where
        t = self.kv[gi][li]
        return CacheView(gi, self.kv_groups[gi].page_tokens, t[0], t[-1], first, writes, states)

    def spare_page(self, group: int) -> int:
        """A page of ``group`` that the manager never hands out."""
        return self.num_pages[group]

    @property
    def spare_slot(self) -> int:
        """A state slot that no request ever holds."""
        return self.max_requests

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + self.state)
