"""What one step needs on the device: the batch's index arrays and scratch.

The reference rebuilds and uploads its index tables layer by layer with
synchronous copies (token/position arrays src/model/gpt2_model.cu:391-392;
token_to_block/offset per layer :214-248; flat block table, offsets and lengths
per layer in decode :544-588: 63 copies per decode step).  Here all of a step's
integers are packed into one pinned buffer and go to the device in one
asynchronous copy; every layer of a cache group reads the same block table.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


def _pad4(n: int) -> int:
    return (n + 3) & ~3


@dataclass
class GroupView:
    """Block tables and cache slots of the step's tokens, for one cache group."""

    block_table: torch.Tensor      # int32 [S, max_pages]
    slot_mapping: torch.Tensor     # int32 [T]; page * page_size + offset of every token
    max_pages: int


@dataclass
class StepLayout:
    """Offsets (in int32 elements) of every section of the packed buffer."""

    T: int
    S: int
    R: int
    max_pages: Tuple[int, ...]
    n_tiles: int = 0
    n_tiles_wide: int = 0
    offsets: Dict[str, int] = field(default_factory=dict)
    total: int = 0

    @classmethod
    def make(cls, T: int, S: int, R: int, max_pages: Sequence[int], n_tiles: int = 0,
             n_tiles_wide: int = 0) -> "StepLayout":
        lay = cls(T, S, R, tuple(max_pages), n_tiles, n_tiles_wide)
        off = 0
        for name, n in (("token_ids", T), ("positions", T), ("token_seq", T), ("logit_rows", R),
                        ("state_slots", S), ("cu_q", S + 1), ("q_start", S), ("ctx_len", S),
                        ("attn_tiles", 3 * n_tiles), ("attn_tiles_wide", 3 * n_tiles_wide)):
            lay.offsets[name] = off
            off += _pad4(n)
        for g, mp in enumerate(max_pages):
            lay.offsets[f"slot_mapping.{g}"] = off
            off += _pad4(T)
            lay.offsets[f"block_table.{g}"] = off
            off += _pad4(S * mp)
        lay.total = off
        return lay

    def key(self):
        return (self.T, self.S, self.R, self.max_pages, self.n_tiles, self.n_tiles_wide)


class Workspace:
    """Scratch tensors by name, allocated once at their largest size.

    ``buf`` returns the first ``rows`` rows of a [max_tokens, cols] buffer, so
    addresses stay the same from step to step (which captured graphs rely on).
    """

    def __init__(self, device, max_tokens: int):
        self.device = device
        self.max_tokens = int(max_tokens)
        self._bufs: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}
        self._logits: Optional[torch.Tensor] = None
        self.version = 0       # bumped when a buffer is replaced by a larger one

    def buf(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, cols, dtype)
        t = self._bufs.get(key)
        if t is None or t.shape[0] < rows:
            cap = max(rows, self.max_tokens)
            t = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self._bufs[key] = t
            self.version += 1
        return t[:rows]

    def zeroed(self, name: str, n: int) -> torch.Tensor:
        """``n`` int32 words that are zero when first handed out; kernels that use them as
        counters leave them zero."""
        key = (name, 0, torch.int32)
        t = self._bufs.get(key)
        if t is None or t.numel() < n:
            t = torch.zeros(max(n, 4096), dtype=torch.int32, device=self.device)
            self._bufs[key] = t
            self.version += 1
        return t[:n]

    def logits(self, rows: int, vocab: int) -> torch.Tensor:
        t = self._logits
        if t is None or t.shape[0] < rows or t.shape[1] != vocab:
            cap = 1
            while cap < rows:
                cap *= 2
            t = torch.empty((cap, vocab), dtype=torch.float32, device=self.device)
            self._logits = t
            self.version += 1
        return t[:rows]


class StepContext:
    """Device views of one step's packed integers, plus host-side facts about it."""

    def __init__(self, layout: StepLayout, dev: torch.Tensor, ws: Workspace, *, q_lens: Sequence[int],
                 q_starts: Sequence[int]):
        self.layout = layout
        self.T, self.S, self.R = layout.T, layout.S, layout.R
        self.ws = ws
        o = layout.offsets

        def sec(name, n):
            return dev[o[name]:o[name] + n]

        self.token_ids = sec("token_ids", self.T)
        self.positions = sec("positions", self.T)
        self.token_seq = sec("token_seq", self.T)
        self.logit_rows = sec("logit_rows", self.R)
        self.state_slots = sec("state_slots", self.S)
        self.cu_q = sec("cu_q", self.S + 1)
        self.q_start = sec("q_start", self.S)
        self.ctx_len = sec("ctx_len", self.S)
        # query tiles of the tensor-core attention: (request index, first flat token, rows)
        self.attn_tiles = sec("attn_tiles", 3 * layout.n_tiles)
        self.n_tiles = layout.n_tiles
        # the same tokens cut into tiles of ATTN_TILE_WIDE rows, for the tcgen05 attention
        self.attn_tiles_wide = sec("attn_tiles_wide", 3 * layout.n_tiles_wide)
        self.n_tiles_wide = layout.n_tiles_wide
        self.groups: List[GroupView] = []
        for g, mp in enumerate(layout.max_pages):
            bt = dev[o[f"block_table.{g}"]:o[f"block_table.{g}"] + self.S * mp].view(self.S, mp)
            self.groups.append(GroupView(block_table=bt, slot_mapping=sec(f"slot_mapping.{g}", self.T), max_pages=mp))
        self.set_host_facts(q_lens, q_starts)

    def set_host_facts(self, q_lens: Sequence[int], q_starts: Sequence[int]) -> None:
        """What the host knows about the step (never read back from the device)."""
        self.q_lens = list(q_lens)
        self.q_starts = list(q_starts)
        self.max_q_len = max(self.q_lens) if self.q_lens else 0
        self.max_ctx_len = max((a + b for a, b in zip(self.q_starts, self.q_lens)), default=0)
        self.decode_only = self.max_q_len == 1


ATTN_TILE = 64      # query rows per tile of csrc/attention_flash.cu and attention_tiled.cu
ATTN_TILE_WIDE = 128     # query rows per tile of csrc/attention_tcgen05.cu


def attention_tiles(q_lens: Sequence[int], q_starts: Optional[Sequence[int]] = None,
                    tile_rows: int = ATTN_TILE) -> List[int]:
    """Cut every request's new tokens into tiles of at most ``tile_rows`` rows: triples of
    (request index in the batch, flat index of the tile's first token, rows).  With the
    positions at which the portions start, the tiles that see the most keys come first,
    so that the longest walks of the attention kernel start earliest."""
    tiles = []
    base = 0
    for s, n in enumerate(q_lens):
        start = 0 if q_starts is None else int(q_starts[s])
        for q0 in range(0, n, tile_rows):
            rows = min(tile_rows, n - q0)
            tiles.append((start + q0 + rows, s, base + q0, rows))
        base += n
    if q_starts is not None:
        tiles.sort(key=lambda t: -t[0])          # stable: equal lengths keep the batch order
    out: List[int] = []
    for _, s, t0, rows in tiles:
        out += [s, t0, rows]
    return out


def pack_step(layout: StepLayout, host: np.ndarray, *, token_ids, positions, token_seq, logit_rows, state_slots,
              cu_q, q_start, ctx_len, slot_mappings, block_tables, attn_tiles=(), attn_tiles_wide=()) -> None:
    """Write every section into the int32 array ``host`` (length >= layout.total)."""
    o = layout.offsets

    def put(name, values):
        a = np.asarray(values, dtype=np.int32).reshape(-1)
        host[o[name]:o[name] + a.size] = a

    put("token_ids", token_ids)
    put("positions", positions)
    put("token_seq", token_seq)
    put("logit_rows", logit_rows)
    put("state_slots", state_slots)
    put("cu_q", cu_q)
    put("q_start", q_start)
    put("ctx_len", ctx_len)
    if layout.n_tiles:
        put("attn_tiles", attn_tiles)
    if layout.n_tiles_wide:
        put("attn_tiles_wide", attn_tiles_wide)
    for g, mp in enumerate(layout.max_pages):
        put(f"slot_mapping.{g}", slot_mappings[g])
        bt = np.zeros((layout.S, mp), dtype=np.int32)
        for s, row in enumerate(block_tables[g]):
            n = min(len(row), mp)
            if n:
                r = np.asarray(row[:n], dtype=np.int32)
                bt[s, :n] = np.where(r < 0, 0, r)
        host[o[f"block_table.{g}"]:o[f"block_table.{g}"] + bt.size] = bt.reshape(-1)
