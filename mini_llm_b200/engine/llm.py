"""The Python entry point: ``LLM(model_dir).generate(prompts, params)``.

It owns what the reference's ServerContext wires together for its server
(src/runtime/server.cpp:92-110: backend, KV allocator, scheduler), without the
TCP front: requests are lists of token ids, responses carry one token each and a
``finished`` flag (include/runtime/response.h:6-17).
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Union

from ..config.base import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .metrics import ServingMetrics
from .request import Request, Response
from .runner import ModelRunner, StepEntry
from .scheduler import PENDING, Scheduler


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", engine: Optional[EngineConfig] = None, **engine_kwargs):
        """``model``: a folder with config.json and model.safetensors.  Keyword
        arguments are fields of EngineConfig (page_size, num_pages, max_num_seqs,
        max_num_batched_tokens, prefill_chunk, admission ...)."""
        if engine is None:
            engine = EngineConfig(dtype=dtype, **engine_kwargs)
        self.engine_config = engine
        self.runner = ModelRunner(model, engine)
        self.config = self.runner.config
        self.scheduler = Scheduler(self.runner.cache, engine, self.runner.max_positions, self.runner.spec.eos_token_id)
        self.sampler = Sampler(self.runner.device, engine.max_num_seqs)
        self._next_id = 0
        self._inflight = None          # (advanced step, sampler ticket, request id -> row) of a step whose tokens are not read yet
        self._held: List[Response] = []     # responses read while aborting, handed out by the next step()
        self.metrics = ServingMetrics()      # arrival, first and last token of every request (host clock)
        self.profile = None                  # a list: step() then times every launch and appends a row per kernel
        self._profile_steps = 0
        self._last_step_shape = None

    # ------------------------------------------------------------------ low level
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        for t in prompt:
            if not (0 <= int(t) < self.runner.vocab_size):
                raise ValueError(f"token id {t} is outside the vocabulary of {self.runner.vocab_size}")
        self.scheduler.add(Request(request_id, list(prompt), params or SamplingParams()))
        self.metrics.arrived(request_id, len(prompt))
        return request_id

    def abort(self, request_id: Hashable) -> bool:
        """Stop a request: its pages and slot are free for others from the next step on.  True if
        the request was still unfinished."""
        if self._inflight is not None:
            self._held += self._finalize()        # tokens that were on their way are still handed out by the next step()
        return self.scheduler.abort(request_id) is not None

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None or bool(self._held)

    def step(self) -> List[Response]:
        """Schedule, launch and sample one step; returns the tokens that became known.

        While only decoding requests are running (``Scheduler.can_run_ahead``) the steps
        overlap: a step is scheduled and launched before the tokens of the one before it
        have been read back, its input tokens are taken from the sampler's device buffer,
        and the host work of a step hides behind the GPU work of the step before.  The
        tokens a call returns are then those of the step launched by the call before.  In
        every other situation (prompts waiting or running, pages short) the tokens are read
        first and a call returns the tokens of its own step, as with
        ``async_scheduling=False``."""
        if self.profile is not None:
            return self._profiled_step()
        out = self._step()
        if out:
            now = self.metrics.clock()
            for r in out:
                self.metrics.token(r.request_id, r.finished, now)
        return out

    def _profiled_step(self) -> List[Response]:
        """One step with every launch timed by CUDA events (needs use_cuda_graphs=False): appends
        (step, kind, requests, tokens, entry point, launches, ms) per kernel entry point to ``self.profile``, the columns
        of the reference's stage timer (include/profiling/stage_timer.cuh:40-101) with the kernel as the stage."""
        from .. import ops
        self._last_step_shape = None
        with ops.time_launches() as tl:
            out = self._step()
        if self._last_step_shape is not None:         # something was launched
            kind, reqs, toks = self._last_step_shape
            for name, n, ms in tl.rows():
                self.profile.append((self._profile_steps, kind, reqs, toks, name.replace("mllm_", ""), n, ms))
            self._profile_steps += 1
        now = self.metrics.clock()
        for r in out:
            self.metrics.token(r.request_id, r.finished, now)
        return out

    def _step(self) -> List[Response]:
        out: List[Response] = self._held
        self._held = []
        ahead = self.engine_config.async_scheduling and self.scheduler.can_run_ahead()
        if self._inflight is not None and not ahead:
            out += self._finalize()
        sched = self.scheduler.schedule()
        launched = None
        if sched.entries:
            rows = self._inflight[2] if self._inflight is not None else {}
            entries = []
            n_tok = sum(len(e.tokens) for e in sched.entries)
            self._last_step_shape = ("decode" if n_tok == len(sched.entries) else
                                     "prefill" if not any(e.is_decode for e in sched.entries) else "mixed",
                                     len(sched.entries), n_tok)
            for e in sched.entries:
                toks = e.tokens
                if e.is_decode and toks[0] == PENDING:
                    toks = [-(rows[e.request.request_id] + 1)]       # still on the device
                entries.append(StepEntry(e.request.request_id, toks, [len(toks) - 1] if e.wants_logits else []))
            logits = self.runner.step(entries, commit=False,
                                      sampled=self.sampler.dev_out if self._inflight is not None else None)
            wanting = [e.request for e in sched.entries if e.wants_logits]
            ticket = self.sampler.launch(logits, wanting) if wanting else None
            adv = self.scheduler.advance(sched)
            launched = (adv, ticket, {r.request_id: i for i, r in enumerate(wanting)})
        if self._inflight is not None:
            out += self._finalize()                # the step before, now that the GPU has the next one queued
        self._inflight = launched
        if launched is not None and not ahead:
            out += self._finalize()
        return out

    def _finalize(self) -> List[Response]:
        adv, ticket, _ = self._inflight
        self._inflight = None
        sampled = self.sampler.fetch(ticket) if ticket is not None else []
        return self.scheduler.resolve(adv, sampled)

    # ------------------------------------------------------------------ generate
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Generated token ids for every prompt, in the order of the prompts."""
        if sampling_params is None:
            sampling_params = SamplingParams()
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        out: Dict[Hashable, List[int]] = {i: [] for i in ids}
        while self.has_unfinished():
            for resp in self.step():
                if resp.request_id in out:
                    out[resp.request_id].append(resp.token)
        return [out[i] for i in ids]
