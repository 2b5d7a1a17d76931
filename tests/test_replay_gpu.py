"""Trace replay against the plain implementation: the same requests whole, with
the last 32 tokens one by one, in portions of changing size, and mixed with other
requests in a pool so small that pages are used again; 32-bit and bfloat16."""
import os

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import CONFIGS, PAGE_SIZE, Replay, assert_close, make_model, oracle_store, random_ids

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 32, 100], "B": [1, 9, 40, 100, 130, 200]}
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def round64(n):
    return (n + 63) // 64 * 64


@pytest.fixture(scope="module", params=[("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    which, dtype = request.param
    d = str(tmp_path_factory.mktemp(f"model_{which}_{dtype}"))
    make_model(d, which, seed=11, dtype=STORE[dtype])
    cfg, w = plain_gpt2.read_model(d)
    reqs = {}
    for i, n in enumerate(LENGTHS[which]):
        ids = random_ids(n, cfg["vocab_size"], 100 + i)
        reqs[f"r{i}"] = (ids, plain_gpt2.forward_logits(cfg, w, ids, oracle_store(dtype)).numpy())
    return dict(which=which, dtype=dtype, dir=d, cfg=cfg, reqs=reqs, page=PAGE_SIZE[which])


def test_whole(setup, tmp_path):
    """Each request alone, whole, all logits wanted."""
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"])
    for rid, (ids, want) in setup["reqs"].items():
        got = rp.step([(rid, ids, range(len(ids)))], end=[rid])
        assert_close(got, want, setup["dtype"], f"whole {rid}")
    assert rp.close() == 0


def test_last_32_one_by_one(setup, tmp_path):
    """Most of the request in one step, the last 32 tokens (or all but one) one by one."""
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"])
    for rid, (ids, want) in setup["reqs"].items():
        n = len(ids)
        head = max(1, n - 32) if n > 1 else 1
        got = [rp.step([(rid, ids[:head], [head - 1])])]
        for i in range(head, n):
            got.append(rp.step([(rid, [ids[i]], [0])]))
        rp.step([], end=[rid])
        assert_close(np.concatenate(got), want[head - 1:], setup["dtype"], f"decode {rid}")
    assert rp.close() == 0


def test_portions_of_changing_size(setup, tmp_path):
    """Prompts cut into portions of 7, 13, 2, 5, 3, 2, 16, 1 ... tokens."""
    sizes = [7, 13, 2, 5, 3, 2, 16, 1, 9, 2, 31]
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"])
    for rid, (ids, want) in setup["reqs"].items():
        pos, k, got = 0, 0, []
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            got.append(rp.step([(rid, ids[pos:pos + n], range(n))]))
            pos += n
        rp.step([], end=[rid])
        assert_close(np.concatenate(got), want, setup["dtype"], f"portions {rid}")
    assert rp.close() == 0


def test_mixed_with_page_reuse(setup, tmp_path):
    """Up to four live requests, portions of some beside decoded tokens of others; the
    pool only holds what is live, so pages of finished requests are used again."""
    reqs = setup["reqs"]
    order = list(reqs)
    # a fixed plan: request -> list of portion sizes (prefill portions, then single tokens)
    plans = {}
    for j, rid in enumerate(order):
        n = len(reqs[rid][0])
        tail = min(n - 1, 6 + 3 * j)
        head = n - tail
        cuts, left, k = [], head, j
        pattern = [13, 2, 7, 24, 3, 50]
        while left > 0:
            c = min(pattern[k % len(pattern)], left)
            cuts.append(c)
            left -= c
            k += 1
        plans[rid] = cuts + [1] * tail
    live, waiting, pos, got = [], list(order), {r: 0 for r in order}, {r: [] for r in order}
    # pool: the four largest requests at once
    need = sum(sorted((round64(len(reqs[r][0])) for r in order), reverse=True)[:4])
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), need, setup["page"])
    step_no = 0
    held = {}
    while waiting or live:
        while waiting and len(live) < 4 and sum(held.values()) + round64(len(reqs[waiting[0]][0])) <= need:
            r = waiting.pop(0)
            live.append(r)
            held[r] = round64(len(reqs[r][0]))
        entries, ending = [], []
        for i, r in enumerate(list(live)):
            if (step_no + i) % 3 == 2 and len(live) > 1:
                continue                     # this request sits the step out
            n = plans[r].pop(0)
            ids = reqs[r][0]
            entries.append((r, ids[pos[r]:pos[r] + n], list(range(n))))
            pos[r] += n
            if not plans[r]:
                ending.append(r)
        out = rp.step(entries, end=ending)
        k = 0
        for r, toks, want in entries:
            got[r].append(out[k:k + len(want)])
            k += len(want)
        for r in ending:
            live.remove(r)
            del held[r]
        step_no += 1
    assert rp.close() == 0
    for r in order:
        assert_close(np.concatenate(got[r]), reqs[r][1], setup["dtype"], f"mixed {r}")
