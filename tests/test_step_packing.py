"""The host side of a step without a GPU: how a batch's integers are laid out in the one buffer
that goes to the device, and how new tokens are cut into attention tiles."""
import random

import numpy as np
import pytest
import torch

from mini_llm_b200.engine.context import (ATTN_TILE, ATTN_TILE_WIDE, StepContext, StepLayout, Workspace,
                                          attention_tiles, pack_step)


def _triples(flat):
    assert len(flat) % 3 == 0
    return [tuple(flat[i:i + 3]) for i in range(0, len(flat), 3)]


@pytest.mark.parametrize("tile_rows", [ATTN_TILE, ATTN_TILE_WIDE, 7])
def test_tiles_cover_every_new_token_once(tile_rows):
    rnd = random.Random(tile_rows)
    for _ in range(50):
        q_lens = [rnd.choice([1, 2, 3, tile_rows - 1, tile_rows, tile_rows + 1, rnd.randint(1, 400)])
                  for _ in range(rnd.randint(1, 6))]
        starts = [rnd.randint(0, 300) for _ in q_lens]
        for q_starts in (None, starts):
            tiles = _triples(attention_tiles(q_lens, q_starts, tile_rows))
            covered = np.zeros(sum(q_lens), dtype=np.int64)
            base = np.concatenate([[0], np.cumsum(q_lens)])
            for s, t0, rows in tiles:
                assert 1 <= rows <= tile_rows
                assert base[s] <= t0 and t0 + rows <= base[s + 1]          # a tile stays inside its request
                assert (t0 - base[s]) % tile_rows == 0                      # and starts at a multiple of the tile
                covered[t0:t0 + rows] += 1
            assert np.all(covered == 1)
            assert len(tiles) == sum((n + tile_rows - 1) // tile_rows for n in q_lens)


def test_tiles_that_see_the_most_keys_come_first():
    q_lens, q_starts = [130, 1, 64, 5], [0, 900, 300, 50]
    tiles = _triples(attention_tiles(q_lens, q_starts, 64))
    base = np.concatenate([[0], np.cumsum(q_lens)])
    seen = [q_starts[s] + (t0 - base[s]) + rows for s, t0, rows in tiles]      # keys the tile's last row sees
    assert seen == sorted(seen, reverse=True)
    # without positions the batch order is kept
    assert [t[0] for t in _triples(attention_tiles(q_lens, None, 64))] == [0, 0, 0, 1, 2, 3]


def test_layout_sections_are_disjoint_and_aligned():
    lay = StepLayout.make(T=37, S=5, R=3, max_pages=[16, 4], n_tiles=6, n_tiles_wide=2)
    spans = []
    sizes = {"token_ids": 37, "positions": 37, "token_seq": 37, "logit_rows": 3, "state_slots": 5, "cu_q": 6,
             "q_start": 5, "ctx_len": 5, "attn_tiles": 18, "attn_tiles_wide": 6, "slot_mapping.0": 37,
             "block_table.0": 5 * 16, "slot_mapping.1": 37, "block_table.1": 5 * 4}
    assert set(lay.offsets) == set(sizes)
    for name, n in sizes.items():
        off = lay.offsets[name]
        assert off % 4 == 0                              # 16-byte aligned sections (int32)
        spans.append((off, off + n))
    spans.sort()
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        assert a1 <= b0
    assert spans[-1][1] <= lay.total
    assert lay.key() != StepLayout.make(37, 5, 3, [16, 4], 6, 3).key()


def test_pack_and_views_round_trip():
    q_lens, q_starts = [3, 1, 70], [10, 40, 0]
    S, T = len(q_lens), sum(q_lens)
    tiles = attention_tiles(q_lens, q_starts)
    wide = attention_tiles(q_lens, q_starts, ATTN_TILE_WIDE)
    lay = StepLayout.make(T, S, 2, [8], len(tiles) // 3, len(wide) // 3)
    host = np.full(lay.total, -7, dtype=np.int32)
    token_ids = np.arange(100, 100 + T)
    positions = np.concatenate([np.arange(a, a + n) for a, n in zip(q_starts, q_lens)])
    token_seq = np.repeat(np.arange(S), q_lens)
    tables = [[[5, 9], [2, -1, 3, 4], [7, 1, 0, 6, 8]]]                 # -1: a page given back (window passed)
    pack_step(lay, host, token_ids=token_ids, positions=positions, token_seq=token_seq, logit_rows=[2, T - 1],
              state_slots=[0, 1, 2], cu_q=[0, 3, 4, T], q_start=q_starts, ctx_len=[13, 41, 70],
              slot_mappings=[np.arange(T) * 2], block_tables=tables, attn_tiles=tiles, attn_tiles_wide=wide)
    ctx = StepContext(lay, torch.from_numpy(host), Workspace(torch.device("cpu"), 8), q_lens=q_lens, q_starts=q_starts)
    assert ctx.token_ids.tolist() == token_ids.tolist()
    assert ctx.positions.tolist() == positions.tolist()
    assert ctx.token_seq.tolist() == token_seq.tolist()
    assert ctx.logit_rows.tolist() == [2, T - 1]
    assert ctx.cu_q.tolist() == [0, 3, 4, T] and ctx.q_start.tolist() == q_starts and ctx.ctx_len.tolist() == [13, 41, 70]
    assert ctx.attn_tiles.tolist() == tiles and ctx.attn_tiles_wide.tolist() == wide
    g = ctx.groups[0]
    assert g.slot_mapping.tolist() == (np.arange(T) * 2).tolist()
    assert g.block_table.shape == (S, 8)
    assert g.block_table[0].tolist() == [5, 9, 0, 0, 0, 0, 0, 0]
    assert g.block_table[1].tolist() == [2, 0, 3, 4, 0, 0, 0, 0]          # a released page reads as page 0, never negative
    assert g.block_table[2].tolist() == [7, 1, 0, 6, 8, 0, 0, 0]
    assert ctx.max_q_len == 70 and ctx.max_ctx_len == 70 and not ctx.decode_only
