"""Serving metrics: the definitions of the reference's offline bench (TTFT, TPOT, E2E, interpolated percentiles)
on a fake clock."""
from mini_llm_b200.engine.metrics import ServingMetrics, mean, percentile


def test_percentile_interpolates_between_ranks():
    xs = [10.0, 20.0, 30.0, 40.0]
    assert percentile(xs, 0) == 10.0 and percentile(xs, 100) == 40.0
    assert percentile(xs, 50) == 25.0                       # rank 1.5
    assert abs(percentile(xs, 90) - 37.0) < 1e-9            # rank 2.7
    assert percentile([], 50) == 0.0 and percentile([7.0], 99) == 7.0
    assert mean([]) == 0.0 and mean([1.0, 3.0]) == 2.0


def test_ttft_tpot_e2e_from_token_times():
    t = [0.0]
    m = ServingMetrics(clock=lambda: t[0])
    m.arrived("a", 5)
    t[0] = 0.010
    m.arrived("b", 9)
    t[0] = 0.050
    m.token("a", False)
    m.token("b", False)
    for k in range(1, 5):                                   # four more tokens for a, 20 ms apart
        t[0] = 0.050 + 0.020 * k
        m.token("a", k == 4)
    t[0] = 0.200
    m.token("b", True)
    rows = {r[0]: r for r in m.rows()}
    assert rows["a"][1:3] == (5, 5) and abs(rows["a"][3] - 50.0) < 1e-9 and abs(rows["a"][4] - 20.0) < 1e-9
    assert abs(rows["a"][5] - 130.0) < 1e-9
    assert rows["b"][2] == 2 and abs(rows["b"][3] - 40.0) < 1e-9 and abs(rows["b"][4] - 150.0) < 1e-9
    s = m.summary()
    assert s["completed"] == 2 and abs(s["total_time_ms"] - 200.0) < 1e-9
    assert abs(s["out_tok_per_s"] - 7 / 0.2) < 1e-9 and abs(s["total_tok_per_s"] - 21 / 0.2) < 1e-9
    assert abs(s["ttft_mean_ms"] - 45.0) < 1e-9 and abs(s["ttft_p50_ms"] - 45.0) < 1e-9
    assert abs(s["e2e_p99_ms"] - (130.0 + 0.99 * 60.0)) < 1e-9


def test_unfinished_requests_do_not_count():
    t = [0.0]
    m = ServingMetrics(clock=lambda: t[0])
    m.arrived(1, 3)
    t[0] = 1.0
    m.token(1, False)
    m.token(99, True)                                       # unknown request: ignored
    assert m.rows() == [] and m.summary()["completed"] == 0 and m.summary()["num_requests"] == 1
