"""Token embedding: x[t] = table[id_t] (+ the position table's row, fused into
the same kernel when the position encoding is an additive table;
src/kernels/embedding.cu:23-43).  The result is the 32-bit residual stream."""
from __future__ import annotations

import torch

from .base import Embedding, ParamSpec, register_part


class TokenEmbedding(Embedding):
    def __init__(self, hidden_size: int, vocab_size: int):
        self.hidden_size = int(hidden_size)
        self.vocab_size = int(vocab_size)

    def param_specs(self):
        return {"table": ParamSpec((self.vocab_size, self.hidden_size), "table")}

    def forward(self, ctx, positions):
        x = ctx.ws.buf("residual", ctx.T, self.hidden_size, torch.float32)
        pos_table = positions.embedding_table() if positions is not None else None
        self.rt.ops.embed(ctx.token_ids, ctx.positions, self.table, pos_table, x)
        return x


register_part("embedding", "token", TokenEmbedding)
