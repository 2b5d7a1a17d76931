"""Generation through the Python entry point against the plain implementation:
greedy and temperature sampling, long decoding, the first tokens of a sequence,
a pool so small that requests are deferred and preempted, the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import CONFIGS, PAGE_SIZE, ROOT, make_model, oracle_store, random_ids

pytestmark = pytest.mark.gpu
STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module", params=[("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    which, dtype = request.param
    d = str(tmp_path_factory.mktemp(f"gen_{which}_{dtype}"))
    make_model(d, which, seed=21, dtype=STORE[dtype])
    cfg, w = plain_gpt2.read_model(d)
    return dict(which=which, dtype=dtype, dir=d, cfg=cfg, w=w, page=PAGE_SIZE[which])


COUNTS = {"float32": [0, 0], "bfloat16": [0, 0]}        # dtype -> [tokens where a near-tie was forgiven, tokens compared]


def follow(cfg, w, prompt, got, store, limit, what, dtype, temperature=0.0, seed=0, rid=0):
    """Every generated token against the plain implementation run on the engine's own prefix: token i must be
    the plain choice after prompt + got[:i].  A difference is accepted only where the plain choice itself hung on
    less than ``limit`` (greedy: the gap between the two logits; sampling: the distance of the uniform draw from
    the edge of the cumulative distribution between the two tokens); such forgiven tokens are counted, and the
    last test of this file bounds their share.  Following the engine's prefix means that a forgiven near-tie does
    not leave the rest of the sequence unchecked."""
    from mini_llm_b200.sampling.params import uniform_for
    ids = list(prompt)
    for i, tok in enumerate(got):
        assert len(ids) <= cfg["n_positions"], f"{what}: token {i} lies beyond the last position"
        row = plain_gpt2.forward_logits(cfg, w, ids, store)[-1]
        if temperature == 0:
            best = plain_gpt2.greedy_token(row)
            margin = float(row[best] - row[tok])
        else:
            u = uniform_for(seed, rid, i)
            best = plain_gpt2.temperature_token(row, temperature, u)
            c = torch.cumsum(torch.softmax(row.double() / temperature, 0), 0)
            lo, hi = min(best, tok), max(best, tok)
            margin = float(torch.min(torch.abs(c[lo:hi] - u))) if lo != hi else 0.0
        COUNTS[dtype][1] += 1
        if tok != best:
            assert margin < limit, f"{what}: token {i} is {tok}, the plain implementation says {best} (margin {margin:.3g})"
            COUNTS[dtype][0] += 1
        ids.append(tok)


def test_greedy_generation(setup):
    import mini_llm_b200 as m
    cfg, w, dtype = setup["cfg"], setup["w"], setup["dtype"]
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], max_tokens=2048, max_num_seqs=4,
                max_num_batched_tokens=64, prefill_chunk=24)
    prompts = [random_ids(n, cfg["vocab_size"], 7 + n) for n in (5, 17, 32, 1, 40)]
    outs = llm.generate(prompts, m.SamplingParams(max_new_tokens=16, ignore_eos=True))
    limit = 1e-3 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        assert len(o) == 16
        follow(cfg, w, p, o, oracle_store(dtype), limit, f"greedy prompt of {len(p)}", dtype)
    assert llm.runner.cache.num_live == 0
    llm.runner.cache.check()


def test_temperature_sampling_follows_the_seeded_draws(setup):
    import mini_llm_b200 as m
    cfg, w, dtype = setup["cfg"], setup["w"], setup["dtype"]
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], max_tokens=2048, max_num_seqs=8,
                max_num_batched_tokens=48, prefill_chunk=13)
    prompts = [random_ids(n, cfg["vocab_size"], 70 + n) for n in (1, 9, 40)]
    ids = [llm.add_request(p, m.SamplingParams(temperature=0.8, seed=1234, max_new_tokens=12, ignore_eos=True))
           for p in prompts]
    outs = {i: [] for i in ids}
    while llm.has_unfinished():
        for r in llm.step():
            outs[r.request_id].append(r.token)
    limit = 1e-5 if dtype == "float32" else 2e-2
    for p, i in zip(prompts, ids):
        assert len(outs[i]) == 12
        follow(cfg, w, p, outs[i], oracle_store(dtype), limit, f"temperature prompt of {len(p)}", dtype,
               temperature=0.8, seed=1234, rid=i)
    # the draw does not depend on the batch: the same request alone gives the same tokens
    llm2 = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], max_tokens=512, max_num_seqs=2)
    rid = llm2.add_request(prompts[1], m.SamplingParams(temperature=0.8, seed=1234, max_new_tokens=12, ignore_eos=True),
                           request_id=ids[1])
    alone = []
    while llm2.has_unfinished():
        alone += [r.token for r in llm2.step()]
    if dtype == "float32":
        assert alone == outs[ids[1]]


def test_long_decoding_to_the_end_of_the_context(setup):
    """A short prompt decoded until the position table is used up."""
    import mini_llm_b200 as m
    cfg, w, dtype = setup["cfg"], setup["w"], setup["dtype"]
    P = cfg["n_positions"]
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], max_tokens=2 * P, max_num_seqs=2)
    prompt = random_ids(3, cfg["vocab_size"], 5)
    out = llm.generate([prompt], m.SamplingParams(max_new_tokens=10 * P, ignore_eos=True))[0]
    assert len(out) == P - 3 + 1                      # every position fed once, one token more
    follow(cfg, w, prompt, out, oracle_store(dtype), 1e-3 if dtype == "float32" else 0.15, "long decode", dtype)


def test_small_pool_defers_and_preempts_but_tokens_stay_the_same(setup):
    import mini_llm_b200 as m
    cfg, dtype, page = setup["cfg"], setup["dtype"], setup["page"]
    prompts = [random_ids(n, cfg["vocab_size"], 300 + n) for n in (20, 33, 12, 27, 8, 30)]
    sp = m.SamplingParams(max_new_tokens=40, ignore_eos=True)
    roomy = m.LLM(setup["dir"], dtype=dtype, page_size=page, max_tokens=4096, max_num_seqs=8)
    want = roomy.generate(prompts, sp)
    tight = m.LLM(setup["dir"], dtype=dtype, page_size=page, num_pages=(33 + 40 + page) // page + 6, max_num_seqs=4,
                  max_num_batched_tokens=32, prefill_chunk=16)
    got = tight.generate(prompts, sp)
    st = tight.scheduler.stats
    assert st.preempted + st.deferred_decode + st.deferred_prefill > 0
    if dtype == "float32":
        assert got == want
    else:
        same = sum(g == w_ for g, w_ in zip(got, want))
        assert same >= len(prompts) - 1        # bfloat16: a near-tie may flip when the batch differs
    tight.runner.cache.check()
    assert tight.runner.cache.num_live == 0 and tight.runner.cache.num_free_pages() == tight.runner.num_pages


def test_running_ahead_gives_the_same_tokens_as_reading_every_step(setup):
    """async_scheduling launches a decode step before the tokens of the one before it are
    read; tokens, finish flags and the cache's state must be those of the step-by-step
    loop, also where an end token arrives while the next step is already running."""
    import mini_llm_b200 as m
    cfg, dtype, page = setup["cfg"], setup["dtype"], setup["page"]
    prompts = [random_ids(n, cfg["vocab_size"], 900 + n) for n in (9, 21, 4, 30)]

    def run(async_on, eos, temperature):
        llm = m.LLM(setup["dir"], dtype=dtype, page_size=page, max_tokens=1024, max_num_seqs=4,
                    async_scheduling=async_on)
        llm.scheduler.eos_token_id = eos
        ids = [llm.add_request(p, m.SamplingParams(temperature=temperature, seed=5, max_new_tokens=14,
                                                   ignore_eos=eos is None)) for p in prompts]
        out = {i: [] for i in ids}
        calls = 0
        while llm.has_unfinished():
            calls += 1
            for r in llm.step():
                assert not (out[r.request_id] and out[r.request_id][-1][1]), "a token after the last one"
                out[r.request_id].append((r.token, r.finished))
        assert llm.runner.cache.num_live == 0
        llm.runner.cache.check()
        assert llm.runner.cache.num_free_pages() == llm.runner.num_pages
        return [out[i] for i in ids], calls

    for temperature in (0.0, 0.7):
        base, _ = run(False, None, temperature)
        ahead, _ = run(True, None, temperature)
        assert ahead == base
        # make the 6th token of the second request the end token
        eos = base[1][5][0]
        base_e, _ = run(False, eos, temperature)
        ahead_e, _ = run(True, eos, temperature)
        assert ahead_e == base_e
        assert base_e[1][-1] == (eos, True) and len(base_e[1]) <= 6
        for o in base_e:
            assert o[-1][1] and all(not f for _, f in o[:-1])


def test_abort_while_running_ahead(setup):
    """A request stopped in the middle of decoding: the others' tokens are what they are without the
    abort, the stopped one hands out no token after the call that stopped it, its pages come back."""
    import mini_llm_b200 as m
    cfg, dtype, page = setup["cfg"], setup["dtype"], setup["page"]
    prompts = [random_ids(n, cfg["vocab_size"], 600 + n) for n in (12, 7, 25)]
    sp = m.SamplingParams(max_new_tokens=12, ignore_eos=True)
    base = m.LLM(setup["dir"], dtype=dtype, page_size=page, max_tokens=512, max_num_seqs=4).generate(prompts, sp)
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=page, max_tokens=512, max_num_seqs=4)
    ids = [llm.add_request(p, sp) for p in prompts]
    out = {i: [] for i in ids}
    stopped_at = None
    while llm.has_unfinished():
        for r in llm.step():
            out[r.request_id].append(r.token)
        if stopped_at is None and len(out[ids[1]]) >= 4:
            assert llm.abort(ids[1])
            assert not llm.abort(ids[1])
            stopped_at = True
    n1 = len(out[ids[1]])
    assert 4 <= n1 <= 6 and out[ids[1]] == base[1][:n1]          # at most the tokens that were already on their way
    assert out[ids[0]] == base[0] and out[ids[2]] == base[2]
    llm.runner.cache.check()
    assert llm.runner.cache.num_live == 0 and llm.runner.cache.num_free_pages() == llm.runner.num_pages


def test_command_line(setup, tmp_path):
    cfg, dtype = setup["cfg"], setup["dtype"]
    p1, p2 = random_ids(6, cfg["vocab_size"], 1), random_ids(11, cfg["vocab_size"], 2)
    f = tmp_path / "prompts.txt"
    f.write_text(" ".join(map(str, p1)) + "\n" + ", ".join(map(str, p2)) + "\n")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "mini_llm"), "--model", setup["dir"], "--dtype", dtype,
           "--kv-block-size", str(setup["page"]), "--total-kv-blocks", "64", "--max-new-tokens", "5", "--ignore-eos",
           "--prompts-file", str(f)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert len(lines) == 2 and all(l.endswith(" [DONE]") for l in lines)
    import mini_llm_b200 as m
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], num_pages=64)
    want = llm.generate([p1, p2], m.SamplingParams(max_new_tokens=5, ignore_eos=True))
    got = [[int(t) for t in l[:-len(" [DONE]")].split()] for l in lines]
    assert got == want


def test_command_line_metrics_and_profile(setup, tmp_path):
    """--metrics prints the serving figures as name,value lines; --profile writes one CSV row per step and kernel entry
    point, timed with CUDA events, and the tokens are the ones of an unprofiled run."""
    cfg, dtype = setup["cfg"], setup["dtype"]
    p1, p2 = random_ids(20, cfg["vocab_size"], 3), random_ids(7, cfg["vocab_size"], 4)
    f = tmp_path / "prompts.txt"
    f.write_text(" ".join(map(str, p1)) + "\n" + " ".join(map(str, p2)) + "\n")
    csv_path = tmp_path / "profile.csv"
    base = [sys.executable, os.path.join(ROOT, "bin", "mini_llm"), "--model", setup["dir"], "--dtype", dtype,
            "--kv-block-size", str(setup["page"]), "--total-kv-blocks", "64", "--max-new-tokens", "6", "--ignore-eos",
            "--prompts-file", str(f)]
    plain = subprocess.run(base, capture_output=True, text=True, timeout=600)
    r = subprocess.run(base + ["--metrics", "--profile", str(csv_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout == plain.stdout
    m = dict(line.split(",") for line in r.stderr.splitlines() if line.count(",") == 1 and not line.startswith("["))
    assert int(m["completed"]) == 2 and float(m["out_tok_per_s"]) > 0
    for name in ("ttft", "tpot", "e2e"):
        assert float(m[f"{name}_mean_ms"]) > 0 and float(m[f"{name}_p50_ms"]) <= float(m[f"{name}_p99_ms"])
    assert float(m["ttft_mean_ms"]) <= float(m["e2e_mean_ms"])
    rows = [l.split(",") for l in csv_path.read_text().splitlines()]
    assert rows[0] == ["step", "kind", "batch_size", "total_tokens", "stage", "launches", "ms"]
    body = rows[1:]
    steps = sorted({int(r_[0]) for r_ in body})
    assert steps == list(range(len(steps))) and len(steps) == 6          # one step for both prompts, five decode steps
    assert body[0][1] == "prefill" and body[0][2:4] == ["2", "27"] and body[-1][1] == "decode" and body[-1][2:4] == ["2", "2"]
    stages = {r_[4] for r_ in body}
    assert "embed" in stages and any(s_.startswith("attention") for s_ in stages) and any(s_.startswith("linear") for s_ in stages)
    assert all(float(r_[6]) > 0 and int(r_[5]) >= 1 for r_ in body)


def test_few_near_ties_had_to_be_forgiven():
    """The tests above accept a token that differs from the plain choice only where that choice was a near-tie.
    All generated tokens were compared (each on the engine's own prefix); here the share of forgiven ones is
    bounded, so that the comparison cannot quietly turn into no comparison: at most one in a hundred in
    float32, one in ten in bfloat16."""
    if COUNTS["float32"][1] == 0 and COUNTS["bfloat16"][1] == 0:
        pytest.skip("the generation tests of this file did not run in this process")
    for dtype, (forgiven, compared) in COUNTS.items():
        if compared:
            assert forgiven <= compared // (100 if dtype == "float32" else 10), f"{dtype}: {forgiven} of {compared} tokens forgiven"
