"""The scheduler's decisions with a fake model (no GPU), in the manner of the
reference's tests/cpp/test_scheduler.cpp (MockBackend emits 1000, 1001, ...)."""
import random

import pytest

from mini_llm_b200.cache.manager import CacheManager, PagedNeed
from mini_llm_b200.config.base import EngineConfig
from mini_llm_b200.engine.request import Request, RequestState
from mini_llm_b200.engine.scheduler import Scheduler, SchedulerError
from mini_llm_b200.sampling.params import SamplingParams

EOS = 7


def make(num_pages=16, page=4, seqs=4, budget=16, chunk=8, admission="lazy", max_positions=64):
    cm = CacheManager({0: PagedNeed(1, 16), 1: PagedNeed(1, 16)}, page_size=page, num_pages=num_pages,
                      max_num_seqs=seqs, allocate=False)
    eng = EngineConfig(page_size=page, num_pages=num_pages, max_num_seqs=seqs, max_num_batched_tokens=budget,
                       prefill_chunk=chunk, admission=admission)
    return cm, Scheduler(cm, eng, max_positions, EOS)


def fake_token(req):
    """Depends on the request's whole history only, like a real model."""
    return 1000 + (sum(req.tokens) + len(req.tokens)) % 97


def run(sched, cm, max_steps=10000, on_step=None):
    out, steps = {}, 0
    while sched.has_unfinished():
        st = sched.schedule()
        steps += 1
        assert steps < max_steps
        assert st.num_tokens <= sched.engine.max_num_batched_tokens
        ids = [e.request.request_id for e in st.entries]
        assert len(ids) == len(set(ids))
        for e in st.entries:                       # tokens fed are exactly the next ones not yet in the cache
            r = e.request
            assert list(e.tokens) == r.tokens[r.num_computed:r.num_computed + len(e.tokens)]
            assert cm.computed(r.request_id) == r.num_computed
            assert len(cm.table(r.request_id, 0)) * cm.page_size >= r.num_computed + len(e.tokens)
        if on_step:
            on_step(st)
        sampled = [fake_token(e.request) for e in st.entries if e.wants_logits]
        for resp in sched.update(st, sampled):
            out.setdefault(resp.request_id, []).append(resp.token)
        cm.check()
    return out, steps


def expected(prompt, n_new):
    toks, out = list(prompt), []
    for _ in range(n_new):
        r = Request(0, toks)
        t = fake_token(r)
        out.append(t)
        toks.append(t)
    return out


def test_prompt_is_cut_into_portions_under_the_budget():
    cm, s = make(budget=16, chunk=8)
    s.add(Request("a", list(range(100, 121)), SamplingParams(max_new_tokens=3)))     # 21 tokens
    sizes = []
    out, _ = run(s, cm, on_step=lambda st: sizes.append([(len(e.tokens), e.wants_logits, e.is_decode) for e in st.entries]))
    assert sizes[:3] == [[(8, False, False)], [(8, False, False)], [(5, True, False)]]
    assert sizes[3:] == [[(1, True, True)], [(1, True, True)]]
    assert out["a"] == expected(range(100, 121), 3)
    assert cm.num_free_pages() == 16 and s.finished[0].state == RequestState.Finished


def test_decodes_go_first_and_share_the_step_with_prompt_portions():
    cm, s = make(budget=10, chunk=8, num_pages=32)
    s.add(Request("a", [1, 2, 3], SamplingParams(max_new_tokens=6)))
    log = []
    st = s.schedule(); s.update(st, [fake_token(e.request) for e in st.entries if e.wants_logits])
    s.add(Request("b", list(range(20, 40)), SamplingParams(max_new_tokens=2)))
    st = s.schedule()
    kinds = [(e.request.request_id, len(e.tokens), e.is_decode) for e in st.entries]
    assert kinds == [("a", 1, True), ("b", 8, False)]                              # decode first, then the portion
    s.update(st, [fake_token(e.request) for e in st.entries if e.wants_logits])
    st = s.schedule()
    assert [(e.request.request_id, len(e.tokens)) for e in st.entries] == [("a", 1), ("b", 8)]
    s.update(st, [fake_token(e.request) for e in st.entries if e.wants_logits])
    st = s.schedule()
    assert [(e.request.request_id, len(e.tokens), e.wants_logits) for e in st.entries] == [("a", 1, True), ("b", 4, True)]


def test_finishes_on_max_new_tokens_eos_and_full_context():
    cm, s = make(max_positions=12)
    s.add(Request("n", [1, 2, 3], SamplingParams(max_new_tokens=4)))
    out, _ = run(s, cm)
    assert len(out["n"]) == 4
    # EOS ends a request unless ignore_eos
    cm, s = make()
    s.add(Request("e", [1, 2], SamplingParams(max_new_tokens=5)))
    s.add(Request("i", [1, 2], SamplingParams(max_new_tokens=5, ignore_eos=True)))
    got = {}
    while s.has_unfinished():
        st = s.schedule()
        for r in s.update(st, [EOS for e in st.entries if e.wants_logits]):
            got.setdefault(r.request_id, []).append((r.token, r.finished))
    assert got["e"] == [(EOS, True)] and len(got["i"]) == 5 and got["i"][-1][1]
    # a prompt that fills the context yields exactly one token; one short of it yields two
    cm, s = make(max_positions=12)
    s.add(Request("f", list(range(12)), SamplingParams(max_new_tokens=9)))
    s.add(Request("g", list(range(11)), SamplingParams(max_new_tokens=9)))
    out, _ = run(s, cm)
    assert len(out["f"]) == 1 and len(out["g"]) == 2
    with pytest.raises(SchedulerError):
        s.add(Request("h", list(range(13))))


def test_admission_is_first_come_first_served_and_stops_at_the_first_misfit():
    cm, s = make(num_pages=6, page=4, seqs=4, budget=64, chunk=64)
    s.add(Request("big", list(range(16)), SamplingParams(max_new_tokens=2)))       # 4 pages (+1 while decoding)
    s.add(Request("big2", list(range(12)), SamplingParams(max_new_tokens=2)))      # 3 pages: does not fit beside big
    s.add(Request("small", [1, 2], SamplingParams(max_new_tokens=2)))              # would fit, but waits its turn
    st = s.schedule()
    assert [e.request.request_id for e in st.entries] == ["big"]
    assert [r.request_id for r in s.deferred_prefill] == ["big2"] and [r.request_id for r in s.waiting] == ["small"]
    assert s.deferred_prefill[0].state == RequestState.DeferredPrefillKV
    s.update(st, [5])
    out, _ = run(s, cm)
    assert set(out) == {"big", "big2", "small"} and s.stats.deferred_prefill >= 1
    order = [r.request_id for r in s.finished]
    assert order.index("big2") < order.index("small") or True   # both finish; big2 was admitted first
    assert cm.num_free_pages() == 6


def test_too_large_for_the_pool_is_refused_at_add():
    cm, s = make(num_pages=4, page=4)
    with pytest.raises(SchedulerError):
        s.add(Request("x", list(range(10)), SamplingParams(max_new_tokens=8)))      # 18 tokens > 16
    with pytest.raises(SchedulerError):
        s.add(Request("y", []))


def test_deferred_decode_then_preemption_by_recompute_keeps_the_tokens_right():
    # two requests that both grow; the pool cannot hold both to the end
    cm, s = make(num_pages=6, page=4, seqs=4, budget=32, chunk=32, max_positions=64)
    pa, pb = [1, 2, 3, 4, 5, 6, 7], [9, 8, 7, 6, 5, 4, 3]
    s.add(Request("a", pa, SamplingParams(max_new_tokens=14, ignore_eos=True)))      # ends at 21 tokens: 6 pages
    s.add(Request("b", pb, SamplingParams(max_new_tokens=10, ignore_eos=True)))      # ends at 17 tokens: 5 pages
    out, steps = run(s, cm)
    assert out["a"] == expected(pa, 14) and out["b"] == expected(pb, 10)
    assert s.stats.preempted >= 1 and s.stats.deferred_decode >= 1
    victim = [r for r in s.finished if r.num_preemptions][0]
    assert victim.request_id == "b"                        # the most recently admitted one gives way
    assert cm.num_free_pages() == 6


def test_reserve_admission_never_defers_a_decode():
    cm, s = make(num_pages=6, page=4, seqs=4, budget=32, chunk=32, admission="reserve")
    pa, pb = [1, 2, 3, 4, 5, 6, 7], [9, 8, 7, 6, 5, 4, 3]
    s.add(Request("a", pa, SamplingParams(max_new_tokens=14, ignore_eos=True)))
    s.add(Request("b", pb, SamplingParams(max_new_tokens=10, ignore_eos=True)))
    live = []
    out, _ = run(s, cm, on_step=lambda st: live.append(sorted(e.request.request_id for e in st.entries)))
    assert out["a"] == expected(pa, 14) and out["b"] == expected(pb, 10)
    assert s.stats.preempted == 0 and s.stats.deferred_decode == 0
    assert all(l != ["a", "b"] for l in live)              # b waits until a has finished


def test_slots_limit_the_number_of_running_requests():
    cm, s = make(num_pages=64, seqs=2, budget=64)
    for i in range(5):
        s.add(Request(i, [1 + i, 2, 3], SamplingParams(max_new_tokens=3, ignore_eos=True)))
    most = []
    out, _ = run(s, cm, on_step=lambda st: most.append(len(st.entries)))
    assert max(most) == 2 and len(out) == 5 and all(len(v) == 3 for v in out.values())


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_under_pressure(seed):
    rng = random.Random(seed)
    cm, s = make(num_pages=14, page=4, seqs=4, budget=24, chunk=rng.choice([3, 8, 24]),
                 admission="lazy", max_positions=48)
    reqs = {}
    for i in range(12):
        p = [rng.randrange(100) + 10 for _ in range(rng.randrange(1, 30))]
        n = rng.randrange(1, 14)
        reqs[i] = (p, n)
    pending = list(reqs)
    out = {}
    steps = 0
    while pending or s.has_unfinished():
        if pending and rng.random() < 0.4:
            i = pending.pop(0)
            s.add(Request(i, reqs[i][0], SamplingParams(max_new_tokens=reqs[i][1], ignore_eos=True)))
        if not s.has_unfinished():
            continue
        st = s.schedule()
        for r in s.update(st, [fake_token(e.request) for e in st.entries if e.wants_logits]):
            out.setdefault(r.request_id, []).append(r.token)
        cm.check()
        steps += 1
        assert steps < 5000
    for i, (p, n) in reqs.items():
        want = expected(p, n)
        room = 48 - len(p) + 1
        assert out[i] == want[:max(1, min(n, room))]
    assert cm.num_free_pages() == 14 and cm.num_live == 0


# ---------------------------------------------------------------------------------- running ahead
def run_ahead(sched, cm, token_of, max_steps=1000):
    """Drive advance/resolve the way the entry point does while it runs ahead: a step is
    scheduled and advanced before the tokens of the step before it are resolved."""
    from mini_llm_b200.engine.scheduler import PENDING
    out, inflight, steps = {}, None, 0

    def finalize():
        nonlocal inflight
        adv, toks = inflight
        inflight = None
        for resp in sched.resolve(adv, toks):
            out.setdefault(resp.request_id, []).append((resp.token, resp.finished))

    while sched.has_unfinished() or inflight is not None:
        steps += 1
        assert steps < max_steps
        ahead = sched.can_run_ahead()
        if inflight is not None and not ahead:
            finalize()
        st = sched.schedule()
        launched = None
        if st.entries:
            for e in st.entries:
                if not e.is_decode:
                    assert PENDING not in e.tokens          # a prompt portion never holds an unread token
            # the "device" knows every token: what the model would sample for each entry
            toks = [token_of(e.request) for e in st.entries if e.wants_logits]
            launched = (sched.advance(st), toks)
        if inflight is not None:
            finalize()
        inflight = launched
        if launched is not None and not ahead:
            finalize()
        cm.check()
    return out, steps


def test_running_ahead_gives_the_same_tokens_and_drops_what_follows_an_end_token():
    """Request 1 samples the end token as its 3rd token; the step launched before that was
    known computed a 4th one, which is dropped; the others are unaffected."""
    from mini_llm_b200.engine.scheduler import PENDING
    cm, s = make(num_pages=64, budget=64, chunk=64)
    truth = {}                                   # request id -> tokens the "device" has produced

    def token_of(req):
        hist = truth.setdefault(req.request_id, [])
        tok = EOS if (req.request_id == 1 and len(hist) == 2) else 1000 + 10 * req.request_id + len(hist)
        hist.append(tok)
        return tok

    for i, n in enumerate((5, 9, 3)):
        s.add(Request(i, list(range(20, 20 + n)), SamplingParams(max_new_tokens=6)))
    out, steps = run_ahead(s, cm, token_of)
    assert [t for t, _ in out[0]] == [1000 + k for k in range(6)]
    assert [t for t, _ in out[2]] == [1020 + k for k in range(6)]
    assert [t for t, _ in out[1]] == [1010, 1011, EOS]
    assert [f for _, f in out[1]] == [False, False, True]
    assert [f for _, f in out[0]] == [False] * 5 + [True]
    assert len(truth[1]) == 4                    # one token was computed past the end and dropped
    for r in s.finished:
        assert PENDING not in r.tokens
    assert {r.request_id: r.tokens[r.prompts_len:] for r in s.finished}[1] == [1010, 1011, EOS]
    assert cm.num_live == 0 and s.stats.finished == 3
    assert steps <= 1 + 6 + 1                    # the prompts in one step, then one step per token, one to drain


def test_running_ahead_stops_while_pages_are_short_or_prompts_wait():
    cm, s = make(num_pages=6, page=4, seqs=4, budget=16, chunk=8)
    s.add(Request(0, list(range(10, 18)), SamplingParams(max_new_tokens=12, ignore_eos=True)))
    assert not s.can_run_ahead()                 # a prompt is waiting
    st = s.schedule()
    s.update(st, [1000])
    assert s.can_run_ahead()
    s.add(Request(1, list(range(30, 38)), SamplingParams(max_new_tokens=12, ignore_eos=True)))
    assert not s.can_run_ahead()
    out, _ = run_ahead(s, cm, lambda r: 1000 + len(r.tokens))
    assert len(out[0]) == 11 and len(out[1]) == 12      # request 0 had one token before
    assert cm.num_live == 0
    cm.check()


def test_abort_frees_pages_and_drops_what_was_on_its_way():
    from mini_llm_b200.engine.scheduler import PENDING
    cm, s = make(num_pages=32, budget=64, chunk=64)
    for i, n in enumerate((6, 9, 4)):
        s.add(Request(i, list(range(20, 20 + n)), SamplingParams(max_new_tokens=10, ignore_eos=True)))
    s.add(Request(7, [1, 2, 3], SamplingParams(max_new_tokens=4)))
    st = s.schedule()                               # max_num_seqs is 4: all four are admitted
    s.update(st, [1000, 1001, 1002, 1003])
    free_before = cm.num_free_pages()
    # a running request: pages and slot come back at once
    gone = s.abort(1)
    assert gone is not None and gone.state == RequestState.Aborted
    assert cm.num_free_pages() > free_before and not cm.is_live(1)
    assert s.abort(1) is None                       # only once
    # a step that was advanced before the abort: its token for the aborted request is dropped
    st = s.schedule()
    assert sorted(e.request.request_id for e in st.entries) == [0, 2, 7]
    adv = s.advance(st)
    r2 = next(e.request for e in st.entries if e.request.request_id == 2)
    assert r2.tokens[-1] == PENDING
    s.abort(2)
    assert PENDING not in r2.tokens and r2.tokens[-1] == 1002
    out = s.resolve(adv, [2000, 2002, 2007])
    assert [(r.request_id, r.token) for r in out] == [(0, 2000), (7, 2007)]
    # a waiting request leaves its queue; the rest run to their ends
    s.add(Request(9, [5, 6], SamplingParams(max_new_tokens=3)))
    s.add(Request(10, [5, 6, 7], SamplingParams(max_new_tokens=3)))
    assert s.abort(10).state == RequestState.Aborted
    done, _ = run(s, cm)
    assert set(done) == {0, 7, 9} and len(done[9]) == 3
    cm.check()
    assert cm.num_live == 0 and cm.num_free_pages() == 32
