"""Arrangements: how a layer's norms, mixer and feed-forward are wired.

"pre_norm" is the reference's block (src/model/gpt2_model.cu:271-365):
x += mixer(norm(x)); x += ff(norm(x)), with the residual stream x in 32-bit.
"""
from __future__ import annotations

from .base import register_part


def _norm(norm, consumer, x, ctx):
    # a consumer that says so gets the norm unevaluated, to fuse it into its first product
    if getattr(consumer, "accepts_lazy_norm", False) and getattr(norm, "supports_lazy", False):
        return norm.forward(x, ctx, lazy=True)
    return norm.forward(x, ctx)


def pre_norm(layer, x, ctx, cache):
    layer.mixer.forward(_norm(layer.mixer_norm, layer.mixer, x, ctx), ctx, cache, x)
    layer.ff.forward(_norm(layer.ff_norm, layer.ff, x, ctx), ctx, x)
    return x


register_part("arrangement", "pre_norm", lambda: pre_norm)
