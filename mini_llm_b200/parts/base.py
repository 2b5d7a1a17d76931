"""Part base classes and the part registries.

A part is built from constants only (its sizes, eps, scale, activation …),
declares the parameters it needs by local name, and gets them bound as device
tensors.  No part knows which model it is in: the checkpoint names of its
parameters live in the ``PartSpec`` that the architecture wrote, not here.

Interfaces (all tensors are CUDA tensors on the engine's stream):

* Norm:          ``forward(x_f32[T,D], ctx, rows=None) -> h[R,D]`` in the activation dtype;
                 ``rows`` (int32 device tensor) gathers those rows of x first.  A norm
                 with ``supports_lazy = True`` also takes ``lazy=True`` and then returns an
                 ``ops.NormedInput`` for consumers with ``accepts_lazy_norm = True``,
                 whose first product fuses the norm into its loads.
* Mixer:         ``forward(h[T,D], ctx, cache, out_accum)``: adds its result into the
                 32-bit residual ``out_accum[T,D]``; ``cache`` is a ``LayerCache``.
                 ``cache_need() -> PagedNeed | StateNeed | None``.
* FeedForward:   ``forward(h[T,D], ctx, out_accum)``: adds into ``out_accum``.
* Positions:     ``embedding_table()``: a [P,D] table added to the token embedding,
                 or None; ``apply_qk(q, k, ctx)``: in-place change of queries/keys
                 (rotations), a no-op for absolute tables; ``max_positions``.
* Embedding:     ``forward(ctx, positions_part) -> x_f32[T,D]``.
* Head:          ``forward(y[R,D], ctx) -> logits_f32[R,V]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional, Tuple


@dataclass
class ParamSpec:
    """``role``: "matrix" and "table" follow the engine dtype (bfloat16 or
    float32); "vector" (norm weights, biases) is always float32; "int" is int32."""

    shape: Tuple[int, ...]
    role: str = "matrix"


class Part:
    category = "part"

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {}

    def kernel_limits(self, dtype: str):
        """Sizes of this part that no kernel of the library takes, as a list of sentences (empty: all
        fine).  Asked once, before any weight is loaded, so that a model that cannot run is refused at
        construction and not at its first step.  ``dtype``: "bfloat16" or "float32"."""
        return []

    def bind(self, params: Dict[str, Any], rt) -> None:
        """Take the loaded parameters (device tensors) and the runtime."""
        self.rt = rt
        for k, v in params.items():
            setattr(self, k, v)


class Norm(Part):
    category = "norm"

    def forward(self, x, ctx, rows=None):  # pragma: no cover
        raise NotImplementedError


class Mixer(Part):
    category = "mixer"

    def cache_need(self):
        return None

    def set_positions(self, positions) -> None:
        self.positions = positions

    def forward(self, h, ctx, cache, out_accum):  # pragma: no cover
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, h, ctx, out_accum):  # pragma: no cover
        raise NotImplementedError


class Positions(Part):
    category = "positions"
    max_positions: Optional[int] = None
    acts_on_qk = False          # True: apply_qk changes queries/keys (a rotation) before keys are cached

    def embedding_table(self):
        return None

    def apply_qk(self, q, k, ctx) -> None:
        return None


class Embedding(Part):
    category = "embedding"

    def forward(self, ctx, positions):  # pragma: no cover
        raise NotImplementedError


class Head(Part):
    category = "head"

    def forward(self, y, ctx):  # pragma: no cover
        raise NotImplementedError


_REGISTRIES: Dict[str, Dict[str, Callable[..., Any]]] = {
    "norm": {}, "mixer": {}, "feed_forward": {}, "positions": {}, "embedding": {}, "head": {},
    "arrangement": {},
}


def register_part(category: str, kind: str, factory: Callable[..., Any], *, replace: bool = False) -> None:
    """Make ``kind`` available to model descriptions.  ``factory(**params)`` builds
    the part (for "arrangement": a function ``f(layer, x, ctx, cache)``)."""
    if category not in _REGISTRIES:
        raise KeyError(f"unknown part category {category!r}; one of {sorted(_REGISTRIES)}")
    if kind in _REGISTRIES[category] and not replace:
        raise KeyError(f"{category} {kind!r} is already registered")
    _REGISTRIES[category][kind] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRIES[category].pop(kind, None)


def get_part_factory(category: str, kind: str):
    reg = _REGISTRIES[category]
    if kind not in reg:
        raise KeyError(f"no {category} named {kind!r}; registered: {sorted(reg)}")
    return reg[kind]


def build_part(category: str, spec) -> Any:
    return get_part_factory(category, spec.kind)(**spec.params)
