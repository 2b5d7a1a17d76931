"""Output heads: logits = y @ W^T in 32-bit, no bias.

``TiedHead`` multiplies by the token embedding's own [V, D] table, which is
already laid out with the contraction dimension contiguous, so no transposed
copy is made (the reference materialises wte_t [D, V] for its GEMM,
src/model/gpt2_model.cu:87-113, 419-428).
"""
from __future__ import annotations

import torch

from .base import Head, ParamSpec, register_part


class TiedHead(Head):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, vocab_size: int):
        self.hidden_size = int(hidden_size)
        self.vocab_size = int(vocab_size)
        self.table = None

    def tie(self, embedding) -> None:
        self.table = embedding.table

    def forward(self, y, ctx):
        out = ctx.ws.logits(y.shape[0], self.vocab_size)
        self.rt.ops.linear(y, self.table, None, out=out)
        return out


class LinearHead(Head):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, vocab_size: int):
        self.hidden_size = int(hidden_size)
        self.vocab_size = int(vocab_size)

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), "matrix")}

    def forward(self, y, ctx):
        out = ctx.ws.logits(y.shape[0], self.vocab_size)
        self.rt.ops.linear(y, self.weight, None, out=out)
        return out


register_part("head", "tied", TiedHead)
register_part("head", "linear", LinearHead)
