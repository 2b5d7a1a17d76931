"""Serving metrics per request: time to first token, time per output token, end-to-end latency.

The definitions are those of the reference's offline serving bench
(benchmarks/serving/offline_gpt2_wmma_bench.cu:542-673): TTFT = first token - arrival,
E2E = last token - arrival, TPOT = (last token - first token) / (output tokens - 1), and
percentiles by linear interpolation between the two nearest ranks (:80-100).  Times are taken
on the host when a request is added and when the entry point hands a token out.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional


def percentile(values: List[float], p: float) -> float:
    """Linear interpolation between the nearest ranks; 0.0 for no values."""
    if not values:
        return 0.0
    xs = sorted(values)
    rank = (p / 100.0) * (len(xs) - 1)
    lo, hi = int(math.floor(rank)), int(math.ceil(rank))
    if lo == hi:
        return xs[lo]
    w = rank - lo
    return xs[lo] * (1.0 - w) + xs[hi] * w


def mean(values: List[float]) -> float:
    return sum(values) / len(values) if values else 0.0


@dataclass
class RequestTimes:
    prompt_len: int
    arrival: float
    first_token: Optional[float] = None
    last_token: Optional[float] = None
    output_len: int = 0
    finished: bool = False

    @property
    def ttft_ms(self) -> float:
        return (self.first_token - self.arrival) * 1e3

    @property
    def e2e_ms(self) -> float:
        return (self.last_token - self.arrival) * 1e3

    @property
    def tpot_ms(self) -> float:
        return (self.last_token - self.first_token) * 1e3 / (self.output_len - 1) if self.output_len > 1 else 0.0


class ServingMetrics:
    def __init__(self, clock=time.perf_counter):
        self.clock = clock
        self.requests: Dict[Hashable, RequestTimes] = {}
        self.start: Optional[float] = None
        self.end: Optional[float] = None

    def arrived(self, request_id: Hashable, prompt_len: int) -> None:
        now = self.clock()
        if self.start is None:
            self.start = now
        self.requests[request_id] = RequestTimes(prompt_len=prompt_len, arrival=now)

    def token(self, request_id: Hashable, finished: bool, now: Optional[float] = None) -> None:
        r = self.requests.get(request_id)
        if r is None:
            return
        now = self.clock() if now is None else now
        if r.first_token is None:
            r.first_token = now
        r.last_token = now
        r.output_len += 1
        r.finished = r.finished or finished
        self.end = now

    def rows(self):
        """(request id, prompt_len, output_len, ttft_ms, tpot_ms, e2e_ms) of every finished request."""
        return [(rid, r.prompt_len, r.output_len, r.ttft_ms, r.tpot_ms, r.e2e_ms)
                for rid, r in self.requests.items() if r.finished and r.first_token is not None]

    def summary(self) -> Dict[str, float]:
        done = [r for r in self.requests.values() if r.finished and r.first_token is not None]
        total_s = (self.end - self.start) if done and self.end is not None else 0.0
        out_tokens = sum(r.output_len for r in done)
        all_tokens = out_tokens + sum(r.prompt_len for r in done)
        s: Dict[str, float] = {"num_requests": len(self.requests), "completed": len(done),
                               "total_time_ms": total_s * 1e3,
                               "req_per_s": len(done) / total_s if total_s > 0 else 0.0,
                               "out_tok_per_s": out_tokens / total_s if total_s > 0 else 0.0,
                               "total_tok_per_s": all_tokens / total_s if total_s > 0 else 0.0}
        for name, vals in (("ttft", [r.ttft_ms for r in done]), ("tpot", [r.tpot_ms for r in done if r.output_len > 1]),
                           ("e2e", [r.e2e_ms for r in done])):
            s[f"{name}_mean_ms"] = mean(vals)
            for p in (50, 90, 95, 99):
                s[f"{name}_p{p}_ms"] = percentile(vals, p)
        return s
