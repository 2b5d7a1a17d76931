"""Arrangements: how a layer's norms, mixer and feed-forward are wired.

"pre_norm" is the reference's block (src/model/gpt2_model.cu:271-365):
x += mixer(norm(x)); x += ff(norm(x)), with the residual stream x in 32-bit.
"""
from __future__ import annotations

from .base import register_part


def pre_norm(layer, x, ctx, cache):
    h = layer.mixer_norm.forward(x, ctx)
    layer.mixer.forward(h, ctx, cache, x)
    h = layer.ff_norm.forward(x, ctx)
    layer.ff.forward(h, ctx, x)
    return x


register_part("arrangement", "pre_norm", lambda: pre_norm)
