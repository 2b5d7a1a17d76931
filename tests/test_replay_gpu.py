"""Trace replay against the plain implementation: the same requests whole, with
the last 32 tokens one by one, in portions of changing size, and mixed with other
requests in a pool so small that pages are used again; 32-bit and bfloat16.

Every shape runs twice: with launches as generation makes them ("on": a step shape that
comes back is captured as a CUDA graph and replayed, so the one-by-one steps are replays and
first sightings run launch by launch) and with every step computed by a replayed graph
("every-step": captured at first sight), so that the logits of the launch mode that serving
uses are graded too, with programmatic dependent launch on in both."""
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


GRAPHS = pytest.mark.parametrize("graphs", ["on", "every-step"])


@GRAPHS
def test_whole(setup, tmp_path, graphs):
    """Each request alone, whole, all logits wanted."""
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"], graphs=graphs)
    for rid, (ids, want) in setup["reqs"].items():
        got = rp.step([(rid, ids, range(len(ids)))], end=[rid])
        assert_close(got, want, setup["dtype"], f"whole {rid}")
    assert rp.close() == 0
    if graphs == "every-step":
        assert rp.stats["graph_replays"] == rp.stats["steps"] > 0


@GRAPHS
def test_last_32_one_by_one(setup, tmp_path, graphs):
    """Most of the request in one step, the last 32 tokens (or all but one) one by one."""
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"], graphs=graphs)
    for rid, (ids, want) in setup["reqs"].items():
        n = len(ids)
        head = max(1, n - 32) if n > 1 else 1
        got = [rp.step([(rid, ids[:head], [head - 1])])]
        for i in range(head, n):
            got.append(rp.step([(rid, [ids[i]], [0])]))
        rp.step([], end=[rid])
        assert_close(np.concatenate(got), want[head - 1:], setup["dtype"], f"decode {rid}")
    assert rp.close() == 0
    # the single-token steps have the same shape again and again: most of them must have been replayed graphs
    assert rp.stats["graph_replays"] >= (rp.stats["steps"] if graphs == "every-step" else rp.stats["steps"] // 2)


@GRAPHS
def test_portions_of_changing_size(setup, tmp_path, graphs):
    """Prompts cut into portions of 7, 13, 2, 5, 3, 2, 16, 1 ... tokens."""
    sizes = [7, 13, 2, 5, 3, 2, 16, 1, 9, 2, 31]
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), round64(256), setup["page"], graphs=graphs)
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


@GRAPHS
@pytest.mark.parametrize("pool_of", [4, 2])
def test_mixed_with_page_reuse(setup, tmp_path, graphs, pool_of):
    """Up to four live requests, portions of some beside decoded tokens of others; the
    pool only holds what is live, so pages of finished requests are used again.  ``pool_of``:
    the pool holds the 4 or the 2 largest requests; with 2 even the configuration with only four
    requests has to hand pages on from a finished request to a new one."""
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
    # pool: the largest requests at once
    need = sum(sorted((round64(len(reqs[r][0])) for r in order), reverse=True)[:pool_of])
    if need >= sum(round64(len(reqs[r][0])) for r in order):
        pytest.skip("this pool holds all requests of the configuration at once: no page would be handed on")
    rp = Replay(setup["dir"], setup["dtype"], str(tmp_path), need, setup["page"], graphs=graphs)
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


# ---------------------------------------------------------------------------------- long prompts, heads of 64
@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def long_setup(request, tmp_path_factory):
    dtype = request.param
    d = str(tmp_path_factory.mktemp(f"model_C_{dtype}"))
    make_model(d, "C", seed=31, dtype=STORE[dtype])
    cfg, w = plain_gpt2.read_model(d)
    reqs = {}
    for i, n in enumerate([700, 300, 513]):
        ids = random_ids(n, cfg["vocab_size"], 500 + i)
        reqs[f"c{i}"] = (ids, plain_gpt2.forward_logits(cfg, w, ids, oracle_store(dtype)).numpy())
    return dict(dtype=dtype, dir=d, cfg=cfg, reqs=reqs, page=PAGE_SIZE["C"])


def test_long_prompts_whole_and_in_long_portions(long_setup, tmp_path):
    """Prompts of several hundred tokens with heads of 64: whole, then in portions whose edges fall inside
    query tiles and key blocks (one of them long enough for the tensor-memory attention kernel on the
    bfloat16 path), then both beside a decoding request."""
    dtype = long_setup["dtype"]
    rp = Replay(long_setup["dir"], dtype, str(tmp_path), round64(704) * 3, long_setup["page"])
    reqs = long_setup["reqs"]
    for rid, (ids, want) in reqs.items():
        n = len(ids)
        places = sorted(set([0, 1, 63, 127, 128, 129, 255, 256, 257, n // 2, n - 2, n - 1]) & set(range(n)))
        got = rp.step([(rid, ids, places)], end=[rid])
        assert_close(got, want[places], dtype, f"whole {rid}")
    # portions: 290 + 300 + the rest, the last logits of every portion and a few inside
    ids, want = reqs["c0"]
    cuts = [0, 290, 590, 700]
    for a, b in zip(cuts[:-1], cuts[1:]):
        places = [0, (b - a) // 2, b - a - 1]
        got = rp.step([("p", ids[a:b], places)])
        assert_close(got, want[[a + p for p in places]], dtype, f"portion {a}:{b}")
    rp.step([], end=["p"])
    # two long portions of different requests in one step beside a single decoded token of a third
    i1, w1 = reqs["c1"]
    i2, w2 = reqs["c2"]
    rp.step([("d", ids[:600], [])])
    got = rp.step([("x", i1[:260], [259]), ("d", [ids[600]], [0]), ("y", i2[:400], [0, 399])])
    assert_close(got, np.stack([w1[259], want[600], w2[0], w2[399]]), dtype, "mixed long portions")
    got = rp.step([("x", i1[260:], [39]), ("y", i2[400:], [112]), ("d", ids[601:603], [1])], end=["x", "y", "d"])
    assert_close(got, np.stack([w1[299], w2[512], want[602]]), dtype, "mixed, second step")
    assert rp.close() == 0


def test_long_portions_take_the_tensor_memory_attention(long_setup):
    """The step function itself: a 600-token portion on the bfloat16 path goes through the tcgen05 attention."""
    if long_setup["dtype"] != "bfloat16":
        pytest.skip("the 32-bit path has its own attention kernels")
    from mini_llm_b200 import ops
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry
    runner = ModelRunner(long_setup["dir"], EngineConfig(dtype="bfloat16", page_size=long_setup["page"], max_tokens=1408,
                                                         max_num_seqs=2, max_num_batched_tokens=1024))
    ids, want = long_setup["reqs"]["c0"]
    before = ops.attention_launches.get("flash_tc", 0)
    runner.add_request("a")
    got = runner.step([StepEntry("a", ids[:600], [0, 300, 599])]).cpu().numpy()
    assert ops.attention_launches.get("flash_tc", 0) == before + long_setup["cfg"]["n_layer"]
    assert_close(got, want[[0, 300, 599]], "bfloat16", "600-token portion")
    ops.check_device_errors()


# ---------------------------------------------------------------------------------- the benchmark's widths
# Two layers at the widths, head counts, vocabulary and positions of GPT-2 small, medium and XL: N = 4800 for
# XL's Q|K|V product, 25 heads, a 50,257-column head whose rows are not 16-byte aligned.
REAL = {"small": (768, 12), "medium": (1024, 16), "xl": (1600, 25)}


def real_config(D, H, n_layer=2):
    return dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=n_layer, n_embd=D, n_head=H, n_inner=4 * D,
                vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                eos_token_id=50256)


@pytest.fixture(scope="module", params=[(s, d) for s in REAL for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def real_setup(request, tmp_path_factory):
    from helpers import make_tensors, write_model
    size, dtype = request.param
    cfg = real_config(*REAL[size])
    d = str(tmp_path_factory.mktemp(f"model_{size}_{dtype}"))
    write_model(d, cfg, make_tensors(cfg, seed=21, sharp=True), STORE[dtype])
    cfg, w = plain_gpt2.read_model(d)
    return dict(size=size, dtype=dtype, dir=d, cfg=cfg, w=w)


def test_real_widths_whole_in_portions_and_one_by_one(real_setup, tmp_path):
    """A 300-token prompt whole, the same as 128 + 172 tokens, then 8 tokens one by one, at a dozen places."""
    dtype, cfg, w = real_setup["dtype"], real_setup["cfg"], real_setup["w"]
    ids = random_ids(308, cfg["vocab_size"], 77)
    places = [0, 1, 15, 16, 127, 128, 129, 255, 256, 299]
    rows = places + list(range(300, 308))
    want = plain_gpt2.logits_at(cfg, w, ids, rows, oracle_store(dtype)).numpy()
    rp = Replay(real_setup["dir"], dtype, str(tmp_path), round64(308) * 2, 16)
    got = rp.step([("w", ids[:300], places)], end=["w"])
    assert_close(got, want[:len(places)], dtype, "whole")
    first = [p for p in places if p < 128]
    got = [rp.step([("p", ids[:128], first)]), rp.step([("p", ids[128:300], [p - 128 for p in places if p >= 128])])]
    assert_close(np.concatenate(got), want[:len(places)], dtype, "128 + 172")
    got = [rp.step([("p", [ids[i]], [0])]) for i in range(300, 308)]
    assert_close(np.concatenate(got), want[len(places):], dtype, "one by one")
    assert rp.close() == 0
    assert rp.stats["graph_replays"] >= 6           # the single-token steps come back with the same shape


MANY = {
    # contexts from 1 to the last position, page and split edges among them; mostly short, so that the
    # plain implementation stays affordable
    "B": [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 130, 200, 255, 256] + list(range(20, 146, 3)),
    "small": [1023, 1024, 641, 513, 512, 257, 129, 128, 127, 65, 64, 17, 16, 1, 2] + list(range(5, 103, 2)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "small"])
def test_a_decode_step_of_40_and_of_64_requests(which, dtype, tmp_path):
    """One decode step with 40 and with 64 live requests, logits of every request against the plain
    implementation: the routes that only large batches take (on the bfloat16 path the tensor-memory product with
    a norm kernel of its own and the cache write in its epilogue; decode attention with one CTA per request and
    head), which the batch-64 point of the benchmark runs."""
    from helpers import make_tensors, write_model
    from mini_llm_b200 import ops
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = CONFIGS["B"] if which == "B" else real_config(*REAL["small"])
    page = PAGE_SIZE["B"] if which == "B" else 16
    d = write_model(str(tmp_path / "m"), cfg, make_tensors(cfg, seed=5, sharp=True), STORE[dtype])
    cfg, w = plain_gpt2.read_model(d)
    lengths = MANY[which]
    assert len(lengths) == 64 and max(lengths) == cfg["n_positions"]
    seqs = [random_ids(n, cfg["vocab_size"], 900 + i) for i, n in enumerate(lengths)]
    want = np.concatenate([plain_gpt2.logits_at(cfg, w, ids, [len(ids) - 1], oracle_store(dtype)).numpy() for ids in seqs])
    pool = sum(-(-n // page) * page for n in lengths)
    runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=page, max_tokens=pool, max_num_seqs=64,
                                         max_num_batched_tokens=2048))
    for count in (40, 64):
        rids = [(count, i) for i in range(count)]
        for r in rids:
            runner.add_request(r)
        batch, used = [], 0
        for r, ids in zip(rids, seqs):                      # the prompts (all but the last token), 2,048 tokens a step
            if len(ids) == 1:
                continue
            if used + len(ids) - 1 > 2048:
                runner.step(batch)
                batch, used = [], 0
            batch.append(StepEntry(r, ids[:-1], []))
            used += len(ids) - 1
        if batch:
            runner.step(batch)
        got = runner.step([StepEntry(r, [ids[-1]], [0]) for r, ids in zip(rids, seqs)]).cpu().numpy()
        ops.check_device_errors()
        assert_close(got, want[:count], dtype, f"decode step of {count}")
        for r in rids:
            runner.finish_request(r)
        runner.cache.check()
