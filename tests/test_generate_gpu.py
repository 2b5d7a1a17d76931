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


def plain_generate(cfg, w, prompt, n_new, store, temperature=0.0, seed=0, rid=0):
    """Greedy or temperature continuation with the margins of every choice."""
    from mini_llm_b200.sampling.params import uniform_for
    ids, out, margins = list(prompt), [], []
    for i in range(n_new):
        if len(ids) > cfg["n_positions"]:
            break
        row = plain_gpt2.forward_logits(cfg, w, ids, store)[-1]
        if temperature == 0:
            tok = plain_gpt2.greedy_token(row)
            top2 = torch.topk(row, 2).values
            margins.append(float(top2[0] - top2[1]))
        else:
            u = uniform_for(seed, rid, i)
            tok = plain_gpt2.temperature_token(row, temperature, u)
            p = torch.softmax(row / temperature, 0)
            c = torch.cumsum(p, 0)
            margins.append(float(torch.min(torch.abs(c - u))))
        out.append(tok)
        ids.append(tok)
    return out, margins


def check_tokens(got, want, margins, limit, what):
    """Equal tokens; a difference is only accepted where the oracle's own choice hung on
    less than ``limit`` (then the rest of the sequence is not comparable)."""
    for i, (g, w_) in enumerate(zip(got, want)):
        if g != w_:
            assert margins[i] < limit, f"{what}: token {i} is {g}, expected {w_} (margin {margins[i]:.3g})"
            return
    assert len(got) == len(want), f"{what}: {len(got)} tokens, expected {len(want)}"


def test_greedy_generation(setup):
    import mini_llm_b200 as m
    cfg, w, dtype = setup["cfg"], setup["w"], setup["dtype"]
    llm = m.LLM(setup["dir"], dtype=dtype, page_size=setup["page"], max_tokens=2048, max_num_seqs=4,
                max_num_batched_tokens=64, prefill_chunk=24)
    prompts = [random_ids(n, cfg["vocab_size"], 7 + n) for n in (5, 17, 32, 1, 40)]
    outs = llm.generate(prompts, m.SamplingParams(max_new_tokens=16, ignore_eos=True))
    limit = 1e-3 if dtype == "float32" else 0.15
    for p, o in zip(prompts, outs):
        want, margins = plain_generate(cfg, w, p, 16, oracle_store(dtype))
        check_tokens(o, want, margins, limit, f"greedy prompt of {len(p)}")
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
        want, margins = plain_generate(cfg, w, p, 12, oracle_store(dtype), temperature=0.8, seed=1234, rid=i)
        check_tokens(outs[i], want, margins, limit, f"temperature prompt of {len(p)}")
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
    want, margins = plain_generate(cfg, w, prompt, len(out), oracle_store(dtype))
    check_tokens(out, want, margins, 1e-3 if dtype == "float32" else 0.15, "long decode")


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
