"""Model: the parts of a ``ModelSpec`` built, bound to weights, and run in order.

The forward pass is the reference's (src/model/gpt2_model.cu:367-453 and
455-689 taken together): embedding, the blocks, the rows whose logits are
wanted gathered and normed, the head.  Here the order of the blocks is a list
(``ModelSpec.schedule``), a block may be named twice, and a run may read
another layer's cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..cache.manager import PagedNeed, StateNeed
from .base import build_part, get_part_factory
from .spec import ModelSpec


@dataclass
class LayerCache:
    """What one run of a layer sees of the cache.

    Paged mixers: ``k_pages``/``v_pages`` [num_pages, kv_heads, page_size, head_dim]
    of the layer, ``group`` (index into ``ctx.groups`` for block table and slot
    mapping).  Mixers with a state: ``state`` [max_num_seqs, *shape], indexed by
    ``ctx.state_slots``.  ``write`` is False when the run borrows another layer's cache.
    """

    group: Optional[int] = None
    k_pages: Any = None
    v_pages: Any = None
    state: Any = None
    write: bool = True


class Layer:
    def __init__(self, spec, hidden_size):
        self.spec = spec
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.mixer = build_part("mixer", spec.mixer)
        self.ff_norm = build_part("norm", spec.ff_norm)
        self.ff = build_part("feed_forward", spec.ff)
        self.arrangement = get_part_factory("arrangement", spec.arrangement)()


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.positions = build_part("positions", spec.positions)
        self.layers: List[Layer] = [Layer(ls, spec.hidden_size) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        for l in self.layers:
            l.mixer.set_positions(self.positions)
        self.rt = None

    def kernel_limits(self, dtype: str) -> List[str]:
        """What the parts report as sizes no kernel takes, each prefixed with the part's label."""
        out: List[str] = []
        for label, _ in self.spec.all_part_specs():
            part = self.part(label)
            check = getattr(part, "kernel_limits", None)
            for msg in (check(dtype) if check is not None else []):
                out.append(f"{label}: {msg}")
        return out

    # -- parts by the labels ModelSpec.all_part_specs() uses
    def part(self, label: str):
        if label.startswith("layers."):
            _, i, name = label.split(".", 2)
            return getattr(self.layers[int(i)], name)
        return getattr(self, label)

    def layer_needs(self) -> Dict[int, object]:
        return {i: l.mixer.cache_need() for i, l in enumerate(self.layers)}

    def finish_binding(self, rt) -> None:
        """Called once all parts have their parameters."""
        self.rt = rt
        if hasattr(self.head, "tie"):
            self.head.tie(self.embedding)

    def layer_cache(self, cache_manager, entry) -> LayerCache:
        owner = entry.cache_of
        write = owner == entry.layer
        need = self.layers[owner].mixer.cache_need()
        if isinstance(need, PagedNeed):
            gi = cache_manager.group_of_layer[owner]
            g = cache_manager.groups[gi]
            li = g.layer_index(owner)
            return LayerCache(group=gi, k_pages=g.pool[li, 0], v_pages=g.pool[li, 1], write=write)
        if isinstance(need, StateNeed):
            return LayerCache(state=cache_manager.states[owner], write=write)
        return LayerCache(write=write)

    def prepare(self, cache_manager) -> None:
        self._caches = [self.layer_cache(cache_manager, e) for e in self.spec.schedule]

    def forward(self, ctx):
        """Run the step's tokens; returns logits [R, vocab] (32-bit) for ctx.logit_rows,
        or None when no logits are wanted."""
        x = self.embedding.forward(ctx, self.positions)
        for entry, cache in zip(self.spec.schedule, self._caches):
            layer = self.layers[entry.layer]
            x = layer.arrangement(layer, x, ctx, cache)
        if ctx.R == 0:
            return None
        if getattr(self.head, "accepts_lazy_norm", False) and getattr(self.final_norm, "supports_lazy", False):
            y = self.final_norm.forward(x, ctx, rows=ctx.logit_rows, lazy=True)
        else:
            y = self.final_norm.forward(x, ctx, rows=ctx.logit_rows)
        return self.head.forward(y, ctx)
