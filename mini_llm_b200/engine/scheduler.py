"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

Same queues and order as the reference's worker loop (src/runtime/scheduler.cpp:
322-356): deferred decodes are retried, running requests decode first (:124-204),
then deferred prompts are retried ahead of waiting ones (:69-87) and admission is
first come first served and stops at the first request that does not fit (:47-67).
Differences: decoded tokens and prompt portions share ONE step (the reference
runs them as separate model calls), a prompt may be cut into portions of at most
``prefill_chunk`` tokens under the step's token budget, and there is no swap to
the CPU (:287-320).

When pages run out:
  * a decoding request that needs a new page and gets none sits the step out in
    ``deferred_decode`` (as :133-145) and is retried next step;
  * a prompt that cannot get pages waits in ``deferred_prefill``;
  * if a whole step can schedule nothing although requests are running, the most
    recently admitted running request is preempted by recompute: its pages and slot
    go back, it returns to the front of the waiting queue with everything it has
    generated so far as its prompt, and admission pauses until a request finishes
    (the reference pauses admission the same way while it swaps, :342-348);
  * a request whose prompt plus max_new_tokens can never fit the pool is refused
    when it is added;
  * with admission="reserve" a request is admitted only when pages for its prompt
    and all its new tokens are free, and takes them at once, so nothing ever stalls.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Tuple

from ..config.base import EngineConfig
from .request import Request, RequestState, Response


class SchedulerError(RuntimeError):
    pass


PENDING = -1      # a generated token whose value has not been read back yet


@dataclass
class ScheduledEntry:
    request: Request
    tokens: List[int]
    wants_logits: bool          # the last of these tokens is followed by a sampled one
    is_decode: bool


@dataclass
class ScheduledStep:
    entries: List[ScheduledEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


@dataclass
class AdvancedStep:
    """A launched step: for every entry that wanted logits, (request, index of the new
    token in request.tokens, finished by count)."""
    step: ScheduledStep
    places: List[Tuple[Request, int, bool]] = field(default_factory=list)


@dataclass
class SchedulerStats:
    steps: int = 0
    tokens: int = 0
    deferred_decode: int = 0
    deferred_prefill: int = 0
    preempted: int = 0
    finished: int = 0
    peak_pages: int = 0


class Scheduler:
    def __init__(self, cache, engine: EngineConfig, max_positions: Optional[int], eos_token_id: Optional[int]):
        self.cache = cache
        self.engine = engine
        self.max_positions = max_positions
        self.eos_token_id = eos_token_id
        self.waiting: Deque[Request] = deque()
        self.deferred_prefill: Deque[Request] = deque()
        self.prefill: List[Request] = []          # admitted, prompt partly in the cache
        self.decode: List[Request] = []           # prompt done, generating
        self.deferred_decode: List[Request] = []
        self.finished: List[Request] = []
        self.admission_paused = False
        self.stats = SchedulerStats()
        self._arrivals = 0

    # ------------------------------------------------------------------ intake
    def add(self, req: Request) -> None:
        n = len(req.tokens)
        if n == 0:
            raise SchedulerError(f"request {req.request_id!r} has an empty prompt")
        if self.max_positions is not None and n > self.max_positions:
            raise SchedulerError(f"request {req.request_id!r}: prompt of {n} tokens exceeds the model's "
                                 f"{self.max_positions} positions")
        total = self._final_length(req)
        for g in self.cache.groups:
            if self.cache.pages_for(total) > g.allocator.num_pages:
                raise SchedulerError(
                    f"request {req.request_id!r} needs {self.cache.pages_for(total)} pages for {total} tokens; "
                    f"the pool has {g.allocator.num_pages}")
        req.state = RequestState.WaitingPrefill
        req.arrival = self._arrivals
        self._arrivals += 1
        self.waiting.append(req)

    def _final_length(self, req: Request) -> int:
        total = req.prompts_len + req.max_new_tokens
        if self.max_positions is not None:
            total = min(total, self.max_positions)
        return max(total, len(req.tokens))

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.deferred_prefill or self.prefill or self.decode or self.deferred_decode)

    @property
    def num_running(self) -> int:
        return len(self.prefill) + len(self.decode) + len(self.deferred_decode)

    # ------------------------------------------------------------------ one step
    def schedule(self) -> ScheduledStep:
        step = self._schedule_once()
        preempted: List[Request] = []
        while not step.entries and self.num_running > 0:
            preempted.append(self._preempt_latest())
            if self.num_running == 0:
                self.admission_paused = False
            step = self._schedule_once()
        step.preempted = preempted
        if not step.entries and self.has_unfinished() and self.num_running == 0:
            head = (self.deferred_prefill or self.waiting)[0]
            raise SchedulerError(f"request {head.request_id!r} cannot be admitted although nothing is running")
        return step

    def _schedule_once(self) -> ScheduledStep:
        e = self.engine
        cm = self.cache
        step = ScheduledStep()
        budget = e.max_num_batched_tokens
        # deferred decodes go back into the decode round (src/runtime/scheduler.cpp:89-100)
        if self.deferred_decode:
            self.decode = sorted(self.decode + self.deferred_decode, key=lambda r: r.arrival)
            self.deferred_decode = []
        # decode first: one token per running request
        still: List[Request] = []
        for req in self.decode:
            if budget <= 0:
                still.append(req)
                continue
            if cm.reserve(req.request_id, 1):
                req.state = RequestState.DecodeRunning
                step.entries.append(ScheduledEntry(req, [req.tokens[-1]], True, True))
                still.append(req)
                budget -= 1
            else:
                req.state = RequestState.DeferredDecodeKV
                self.deferred_decode.append(req)
                self.stats.deferred_decode += 1
        self.decode = still
        # prompts already admitted go on with their next portion
        for req in self.prefill:
            if budget <= 0:
                break
            budget -= self._portion(req, budget, step)
        # then admission: deferred prompts first, then waiting ones; stop at the first that does not fit
        if not self.admission_paused:
            while budget > 0 and (self.deferred_prefill or self.waiting):
                src = self.deferred_prefill if self.deferred_prefill else self.waiting
                req = src[0]
                if not self._admit(req, budget):
                    if src is self.waiting:
                        self.waiting.popleft()
                        req.state = RequestState.DeferredPrefillKV
                        self.deferred_prefill.append(req)
                        self.stats.deferred_prefill += 1
                    break
                src.popleft()
                req.state = RequestState.PrefillRunning
                self.prefill.append(req)
                budget -= self._portion(req, budget, step)
        return step

    def _admit(self, req: Request, budget: int) -> bool:
        cm = self.cache
        if not cm.can_admit():
            return False
        first = min(len(req.tokens), self.engine.prefill_chunk, budget)
        need = self._final_length(req) if self.engine.admission == "reserve" else first
        pages = cm.pages_for(need)
        if not all(g.allocator.can_allocate(pages) for g in cm.groups):
            return False
        cm.admit(req.request_id)
        req.num_computed = 0
        if self.engine.admission == "reserve":
            ok = cm.reserve(req.request_id, need)
            assert ok
        return True

    def _portion(self, req: Request, budget: int, step: ScheduledStep) -> int:
        """Schedule the next portion of an admitted prompt; returns its length (0 if no pages)."""
        left = len(req.tokens) - req.num_computed
        n = min(left, self.engine.prefill_chunk, budget)
        if n <= 0:
            return 0
        if not self.cache.reserve(req.request_id, n):
            return 0
        toks = req.portion(req.num_computed, req.num_computed + n)
        step.entries.append(ScheduledEntry(req, toks, n == left, False))
        return n

    def _preempt_latest(self) -> Request:
        running = self.prefill + self.decode + self.deferred_decode
        victim = max(running, key=lambda r: r.arrival)
        for q in (self.prefill, self.decode, self.deferred_decode):
            if victim in q:
                q.remove(victim)
        self.cache.release(victim.request_id)
        victim.num_computed = 0
        victim.num_preemptions += 1
        victim.state = RequestState.WaitingPrefill
        self.waiting.appendleft(victim)
        self.admission_paused = len(running) > 1
        self.stats.preempted += 1
        return victim

    # ------------------------------------------------------------------ after the model ran
    def advance(self, step: ScheduledStep) -> "AdvancedStep":
        """The step has been launched: its tokens are held by the cache, and every entry that
        wanted logits gets a place for its new token (``PENDING`` until ``resolve`` fills it
        in).  What depends on the count of tokens alone is decided here: a request that has
        reached max_new_tokens or the model's last position finishes and frees its pages,
        although the value of its last token is not known yet.  The next step can be
        scheduled on this state; a token that turns out to end its request is found by
        ``resolve``."""
        adv = AdvancedStep(step)
        self.stats.steps += 1
        self.stats.tokens += step.num_tokens
        for en in step.entries:
            req = en.request
            self.cache.commit(req.request_id, len(en.tokens))
            req.num_computed += len(en.tokens)
            if not en.wants_logits:
                continue
            index = len(req.tokens)
            req.tokens.append(PENDING)
            finished = req.isfinish()
            if self.max_positions is not None and len(req.tokens) >= self.max_positions + 1:
                finished = True             # the new token has no position left to be fed at
            adv.places.append((req, index, finished))
            if not en.is_decode:
                self.prefill.remove(req)
            if finished:
                if en.is_decode:
                    self.decode.remove(req)
                self._finish(req)
            else:
                req.state = RequestState.DecodeReady
                if not en.is_decode:
                    self.decode.append(req)
        for g in self.cache.groups:
            self.stats.peak_pages = max(self.stats.peak_pages, g.allocator.peak_in_use)
        return adv

    def resolve(self, adv: "AdvancedStep", sampled: List[int]) -> List[Response]:
        """``sampled``: one token for every entry of the step that wanted logits, in order.
        Fills them in; a request whose token is the end-of-sequence token finishes here, and
        what a later step (launched before this was known) computed for it is dropped."""
        out: List[Response] = []
        if len(sampled) != len(adv.places):
            raise SchedulerError(f"{len(adv.places)} tokens expected, {len(sampled)} given")
        for (req, index, finished), tok in zip(adv.places, sampled):
            if req.ended_at is not None and index > req.ended_at:
                continue                        # computed after the request's last token: dropped
            tok = int(tok)
            req.tokens[index] = tok
            if not req.params.ignore_eos and self.eos_token_id is not None and tok == self.eos_token_id:
                req.ended_at = index
                del req.tokens[index + 1:]
                if req.state != RequestState.Finished:
                    if req in self.decode:
                        self.decode.remove(req)
                    if req in self.deferred_decode:
                        self.deferred_decode.remove(req)
                    self._finish(req)
                finished = True
            out.append(Response(req.request_id, tok, finished))
        return out

    def update(self, step: ScheduledStep, sampled: List[int]) -> List[Response]:
        """advance and resolve in one call, for a caller that has the tokens at hand."""
        return self.resolve(self.advance(step), sampled)

    def abort(self, request_id: Hashable) -> Optional[Request]:
        """Take a request out wherever it stands: waiting requests just leave their queue, running
        ones give back their pages and their slot.  Returns the request (state Aborted), or None
        if no unfinished request has this id.  Tokens of a step that was launched before the
        abort and is resolved after it are dropped."""
        for q in (self.waiting, self.deferred_prefill):
            for req in q:
                if req.request_id == request_id:
                    q.remove(req)
                    req.state = RequestState.Aborted
                    return req
        for q in (self.prefill, self.decode, self.deferred_decode):
            for req in q:
                if req.request_id == request_id:
                    q.remove(req)
                    self.cache.release(req.request_id)
                    # what an unresolved step computed for it is dropped; unread tokens leave the list
                    while req.tokens and req.tokens[-1] == PENDING:
                        req.tokens.pop()
                    req.ended_at = len(req.tokens) - 1
                    req.state = RequestState.Aborted
                    self.admission_paused = False
                    return req
        return None

    def _finish(self, req: Request) -> None:
        self.cache.release(req.request_id)
        req.state = RequestState.Finished
        self.finished.append(req)
        self.stats.finished += 1
        self.admission_paused = False

    def can_run_ahead(self) -> bool:
        """True when the next step can be scheduled before the last one's tokens are known:
        only decoding requests, and a free page in every group for each of them, so that
        nothing is admitted, cut, deferred or preempted on a token that is still pending."""
        if self.waiting or self.deferred_prefill or self.prefill or self.deferred_decode:
            return False
        n = len(self.decode)
        return all(g.allocator.num_free >= n for g in self.cache.groups)
