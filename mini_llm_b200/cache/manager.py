"""The cache manager: pages of keys and values per request, and state slots.

Layers are put into groups by what they need of the cache (how many key/value
heads of which size, all keys or a window of them); every group has its own
page pool, allocator and one block table per request.  Next to the pages each
live request owns a slot id: its row in the per-layer state arenas of mixers
that keep a fixed-size state.

What the reference does with the same job: one block table per layer per
request, all from one pool (src/runtime/real_kv_allocator.cu:112-177),
all-or-nothing admission of a whole prompt (:112-139), one block per layer when
a decode crosses a block edge (:141-168), everything returned when the request
finishes (:170-177).  Here a reservation covers any number of new tokens, so
portions of prompts and decoded tokens go the same way.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .pages import PageAllocator, PageError

RELEASED = -1   # block-table entry of a page that a window has passed


@dataclass(frozen=True)
class PagedNeed:
    """A mixer that keeps keys and values of past tokens in pages."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None      # None: every past token stays visible


@dataclass(frozen=True)
class StateNeed:
    """A mixer that keeps a state of fixed size per request."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


class CacheGroup:
    """Layers with the same PagedNeed: one pool, one allocator, one table per request."""

    def __init__(self, index: int, need: PagedNeed, layers: List[int], num_pages: int, page_size: int):
        self.index = index
        self.need = need
        self.layers = list(layers)
        self.page_size = page_size
        self.allocator = PageAllocator(num_pages)
        self.tables: Dict[Hashable, List[int]] = {}
        self.pool = None            # device tensor [len(layers), 2, num_pages, kv_heads, page_size, head_dim]

    def layer_index(self, layer: int) -> int:
        return self.layers.index(layer)

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.layers) * self.need.kv_heads * self.need.head_dim * element_size


@dataclass
class _Live:
    slot: int
    computed: int = 0                       # tokens whose keys/values/state are in the cache
    first_kept: Dict[int, int] = field(default_factory=dict)   # group -> first page index still held


class CacheManager:
    def __init__(self, layer_needs: Dict[int, object], *, page_size: int, num_pages, max_num_seqs: int,
                 dtype=None, device=None, allocate: bool = True):
        """``layer_needs``: layer index -> PagedNeed | StateNeed | None.
        ``num_pages``: pages of every group, or a dict group-key -> pages."""
        import torch

        self.page_size = page_size
        self.max_num_seqs = max_num_seqs
        self.groups: List[CacheGroup] = []
        self.group_of_layer: Dict[int, int] = {}
        self.state_layers: Dict[int, StateNeed] = {}
        by_need: Dict[PagedNeed, List[int]] = {}
        for layer in sorted(layer_needs):
            need = layer_needs[layer]
            if need is None:
                continue
            if isinstance(need, PagedNeed):
                by_need.setdefault(need, []).append(layer)
            elif isinstance(need, StateNeed):
                self.state_layers[layer] = need
            else:
                raise TypeError(f"layer {layer}: unknown cache need {need!r}")
        for need, layers in by_need.items():
            n = num_pages[need] if isinstance(num_pages, dict) else int(num_pages)
            g = CacheGroup(len(self.groups), need, layers, n, page_size)
            for l in layers:
                self.group_of_layer[l] = g.index
            self.groups.append(g)
        self._live: Dict[Hashable, _Live] = {}
        self._free_slots: List[int] = list(range(max_num_seqs - 1, -1, -1))
        self.states: Dict[int, "torch.Tensor"] = {}
        self.dtype = dtype
        self.device = device
        if allocate:
            for g in self.groups:
                g.pool = torch.zeros(
                    (len(g.layers), 2, g.allocator.num_pages, g.need.kv_heads, page_size, g.need.head_dim),
                    dtype=dtype, device=device)
            for layer, need in self.state_layers.items():
                self.states[layer] = torch.zeros((max_num_seqs,) + tuple(need.shape),
                                                 dtype=getattr(torch, need.dtype), device=device)

    # ------------------------------------------------------------------ requests
    def is_live(self, req) -> bool:
        return req in self._live

    @property
    def num_live(self) -> int:
        return len(self._live)

    def can_admit(self) -> bool:
        return bool(self._free_slots)

    def admit(self, req) -> int:
        """Give the request a state slot (zeroed) and empty block tables."""
        if req in self._live:
            raise PageError(f"request {req!r} is already live")
        if not self._free_slots:
            raise PageError("no state slot free")
        slot = self._free_slots.pop()
        self._live[req] = _Live(slot=slot, first_kept={g.index: 0 for g in self.groups})
        for g in self.groups:
            g.tables[req] = []
        for t in self.states.values():
            t[slot].zero_()
        return slot

    def slot(self, req) -> int:
        return self._live[req].slot

    def computed(self, req) -> int:
        return self._live[req].computed

    def table(self, req, group: int) -> List[int]:
        return self.groups[group].tables[req]

    # ------------------------------------------------------------------ pages
    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def pages_missing(self, req, n_new: int) -> Dict[int, int]:
        """Pages each group still lacks to hold tokens [0, computed + n_new)."""
        lv = self._live[req]
        total = self.pages_for(lv.computed + n_new)
        return {g.index: max(0, total - len(g.tables[req])) for g in self.groups}

    def can_reserve(self, req, n_new: int) -> bool:
        miss = self.pages_missing(req, n_new)
        return all(self.groups[gi].allocator.can_allocate(n) for gi, n in miss.items())

    def reserve(self, req, n_new: int) -> bool:
        """Pages for the next n_new tokens in every group, or none at all."""
        total = (self._live[req].computed + n_new + self.page_size - 1) // self.page_size
        if all(len(g.tables[req]) >= total for g in self.groups):
            return True                              # the common decode case: the last page still has room
        miss = self.pages_missing(req, n_new)
        if not all(self.groups[gi].allocator.can_allocate(n) for gi, n in miss.items()):
            return False
        for gi, n in miss.items():
            if n:
                g = self.groups[gi]
                g.tables[req].extend(g.allocator.allocate(n))
        return True

    def commit(self, req, n_new: int) -> None:
        """n_new more tokens are in the cache; pages a window has passed go back."""
        lv = self._live[req]
        lv.computed += n_new
        for g in self.groups:
            if len(g.tables[req]) < self.pages_for(lv.computed):
                raise PageError(f"request {req!r}: {lv.computed} tokens committed but only "
                                f"{len(g.tables[req])} pages reserved in group {g.index}")
            w = g.need.window
            if w is None:
                continue
            # the next query stands at position >= computed and sees keys >= computed - w + 1
            first_needed = max(0, lv.computed - w + 1) // self.page_size
            tab = g.tables[req]
            gone = []
            for p in range(lv.first_kept[g.index], min(first_needed, len(tab))):
                if tab[p] != RELEASED:
                    gone.append(tab[p])
                    tab[p] = RELEASED
            if gone:
                g.allocator.free(gone)
            lv.first_kept[g.index] = max(lv.first_kept[g.index], min(first_needed, len(tab)))

    def release(self, req) -> None:
        """The request ends: its pages and its slot go back."""
        if req not in self._live:
            raise PageError(f"request {req!r} is not live (released twice?)")
        lv = self._live.pop(req)
        for g in self.groups:
            g.allocator.free([p for p in g.tables.pop(req) if p != RELEASED])
        self._free_slots.append(lv.slot)

    def slots_for(self, req, group: int, start: int, n: int) -> List[int]:
        """Flat cache slot (page * page_size + offset) of positions start..start+n-1."""
        tab = self.groups[group].tables[req]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            page = tab[pos // ps]
            if page == RELEASED:
                raise PageError(f"request {req!r}: position {pos} lies in a released page")
            out.append(page * ps + pos % ps)
        return out

    # ------------------------------------------------------------------ checks
    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.num_free

    def check(self) -> None:
        """No page lost, none held twice; slots likewise."""
        for g in self.groups:
            g.allocator.check()
            held = [p for t in g.tables.values() for p in t if p != RELEASED]
            if len(held) != len(set(held)):
                raise PageError(f"group {g.index}: a page is held by two requests")
            for p in held:
                if not g.allocator.is_in_use(p):
                    raise PageError(f"group {g.index}: page {p} is held but marked free")
            if len(held) != g.allocator.num_in_use:
                raise PageError(f"group {g.index}: {g.allocator.num_in_use} pages in use, {len(held)} held")
        slots = [lv.slot for lv in self._live.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise PageError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise PageError("a state slot is lost")
