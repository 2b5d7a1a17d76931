"""Position encodings.

``LearnedPositions``: a [P, D] table added to the token embedding at the
token's absolute index in its request (src/kernels/embedding.cu:23-43; the
reference counts positions from 0 per request, src/model/gpt2_model.cu:379-386,
and feeds a decoded token at position len-1, :466-469).  The table's height
bounds the context.
"""
from __future__ import annotations

from .base import ParamSpec, Positions, register_part


class LearnedPositions(Positions):
    def __init__(self, hidden_size: int, max_positions: int):
        self.hidden_size = int(hidden_size)
        self.max_positions = int(max_positions)

    def param_specs(self):
        return {"table": ParamSpec((self.max_positions, self.hidden_size), "table")}

    def embedding_table(self):
        return self.table


class NoPositions(Positions):
    """No position information at all (for mixers that need none)."""

    def __init__(self, hidden_size: int = 0):
        self.max_positions = None


register_part("positions", "learned", LearnedPositions)
register_part("positions", "none", NoPositions)
