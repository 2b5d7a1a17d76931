"""The step function: one batch of (request, its next tokens) through the model.

The reference has two entry points, GPT2Model::prefill for whole prompts from
position 0 (src/model/gpt2_model.cu:367-453) and GPT2Model::decode for one token
per request (:455-689), never mixed.  ``ModelRunner.step`` takes any mix: portions
of prompts of any length beside single decoded tokens.  It runs only the tokens
it is given, reads everything older from the cache, and returns the logits at
the wanted places.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from ..config.base import ConfigError, EngineConfig, ModelConfig, get_architecture, load_config
from ..parts.model import Model
from ..weights.loader import load_weights
from .context import ATTN_TILE_WIDE, StepContext, StepLayout, Workspace, attention_tiles, pack_step


class StepError(RuntimeError):
    pass


class OutOfPages(StepError):
    """The cache has no pages left for the tokens of this step."""


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and where logits are wanted."""

    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)     # indices into ``tokens``


@dataclass
class Runtime:
    dtype: torch.dtype
    device: torch.device
    ops: object = ops

    @property
    def act_dtype(self) -> torch.dtype:
        return self.dtype


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class ModelRunner:
    def __init__(self, model_dir: str, engine: Optional[EngineConfig] = None):
        self.engine = engine or EngineConfig()
        self.config: ModelConfig = load_config(model_dir)
        arch = get_architecture(self.config.architecture)
        self.spec = arch.build_spec(self.config)
        self.model = Model(self.spec)
        # sizes no kernel takes are refused here, before a device is touched, a weight loaded or a pool allocated
        problems = list(dict.fromkeys(m.split(": ", 1)[1] for m in self.model.kernel_limits(self.engine.dtype)))
        if problems:
            raise ConfigError(f"{model_dir}: this model cannot run on the kernel library: " + "; ".join(problems))
        if not torch.cuda.is_available():
            raise StepError("no CUDA device: this engine has no CPU path")
        self.device = torch.device(self.engine.device)
        torch.cuda.set_device(self.device)
        ops.library()       # build/load now: fail early and loudly
        ops.set_pdl(self.engine.use_pdl)
        self.rt = Runtime(dtype=torch.bfloat16 if self.engine.dtype == "bfloat16" else torch.float32,
                          device=self.device)
        load_weights(self.model, self.spec, model_dir, self.rt)
        self.vocab_size = self.spec.vocab_size
        self.max_positions = self.spec.max_positions
        self._make_cache()
        self.model.prepare(self.cache)
        self.ws = Workspace(self.device, self.engine.max_num_batched_tokens)
        self._host = [None, None]
        self._host_events = [None, None]
        self._host_turn = 0
        self._dev: Optional[torch.Tensor] = None
        self._ctx_cache: Dict[tuple, StepContext] = {}
        self.steps_run = 0
        # CUDA graphs of decode-only steps, by the step's shape
        self._graphs: Dict[tuple, object] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_families = set()
        self._graph_version = None
        self.graph_replays = 0
        self.graph_kernels: Dict[tuple, int] = {}
        # a part that reads device data on the host while it runs sets graph_safe = False
        self._graph_ok = all(getattr(self.model.part(label), "graph_safe", True)
                             for label, _ in self.spec.all_part_specs())
        self._capture_at_once = self.engine.graph_capture == "at_once"
        if self._capture_at_once and self.cache.state_layers:
            raise StepError("graph_capture='at_once' runs a new step shape twice; a mixer with a state of its own "
                            "would advance it twice")

    # ------------------------------------------------------------------ set-up
    def _make_cache(self) -> None:
        e = self.engine
        needs = self.model.layer_needs()
        probe = CacheManager(needs, page_size=e.page_size, num_pages=0, max_num_seqs=1, allocate=False)
        es = _element_size(self.rt.dtype)
        if e.num_pages is not None:
            num_pages = int(e.num_pages)
        elif e.max_tokens is not None:
            num_pages = (int(e.max_tokens) + e.page_size - 1) // e.page_size
        else:
            per_token = sum(g.bytes_per_token(es) for g in probe.groups) or 1
            free, _ = torch.cuda.mem_get_info(self.device)
            tokens = int(free * e.memory_fraction) // per_token
            limit = e.max_num_seqs * (self.max_positions or 1 << 20)
            tokens = max(e.page_size, min(tokens, limit))
            num_pages = (tokens + e.page_size - 1) // e.page_size
        self.cache = CacheManager(needs, page_size=e.page_size, num_pages=num_pages, max_num_seqs=e.max_num_seqs,
                                  dtype=self.rt.dtype, device=self.device)
        self.num_pages = num_pages

    def _staging(self, n: int):
        i = self._host_turn
        self._host_turn ^= 1
        if self._host[i] is None or self._host[i].numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            self._host[i] = torch.empty(cap, dtype=torch.int32, pin_memory=True)
            self._host_events[i] = torch.cuda.Event()
        else:
            self._host_events[i].synchronize()      # the copy that last used this buffer is done
        if self._dev is None or self._dev.numel() < n:
            cap = max(4096, 1 << (n - 1).bit_length())
            self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self.ws.version += 1
        return i, self._host[i]

    # ------------------------------------------------------------------ requests
    def add_request(self, req) -> None:
        self.cache.admit(req)

    def has_request(self, req) -> bool:
        return self.cache.is_live(req)

    def finish_request(self, req) -> None:
        self.cache.release(req)

    def computed(self, req) -> int:
        return self.cache.computed(req)

    # ------------------------------------------------------------------ the step
    def prepare_step(self, entries: Sequence[StepEntry], sampled: Optional[torch.Tensor] = None) -> StepContext:
        """Reserve pages, pack the step's integers, start their copy to the device.  With
        ``sampled`` (the device buffer of the last sampling launch) a token may be given as
        -(row + 1): the value that launch wrote to that row, filled in on the device."""
        cm = self.cache
        pending = False
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        toks: List[np.ndarray] = []
        for en in entries:
            if en.req in seen:
                raise StepError(f"request {en.req!r} appears twice in one step")
            seen.add(en.req)
            if not cm.is_live(en.req):
                raise StepError(f"request {en.req!r} is not live (add_request first)")
            n = len(en.tokens)
            if n == 0:
                raise StepError(f"request {en.req!r} brings no tokens")
            if n == 1:                                   # a decoded token: no array needed to check it
                arr = (int(en.tokens[0]),)
                lo = hi = arr[0]
            else:
                arr = np.asarray(en.tokens, dtype=np.int64).reshape(-1)
                lo, hi = int(arr.min()), int(arr.max())
            start = cm.computed(en.req)
            if self.max_positions is not None and start + n > self.max_positions:
                raise StepError(f"request {en.req!r}: {start + n} tokens exceed the model's {self.max_positions} positions")
            if lo < 0 and sampled is not None and lo >= -int(sampled.numel()):
                pending = True
                lo = 0
            if lo < 0 or hi >= self.vocab_size:
                bad = next(int(t) for t in en.tokens if not (0 <= int(t) < self.vocab_size))
                raise StepError(f"request {en.req!r}: token id {bad} is outside the vocabulary of {self.vocab_size}")
            for w in en.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {en.req!r}: wanted place {w} is outside its {n} tokens")
            toks.append(arr)
        for en, arr in zip(entries, toks):
            if not cm.reserve(en.req, len(arr)):
                raise OutOfPages(f"no pages left for {len(arr)} tokens of request {en.req!r} "
                                 f"({[g.allocator.num_free for g in cm.groups]} free)")
        S = len(entries)
        ps = cm.page_size
        q_lens = [len(a) for a in toks]
        q_start = [cm.computed(en.req) for en in entries]
        ctx_len = [a + b for a, b in zip(q_start, q_lens)]
        slots = [cm.slot(en.req) for en in entries]
        cu_q = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu_q[1:])
        T = int(cu_q[-1])
        ng = len(cm.groups)
        tables = [[cm.table(en.req, g) for en in entries] for g in range(ng)]
        if T == S:                                   # a decode step: one token each, plain integers are quickest
            token_ids = np.fromiter((a[0] for a in toks), dtype=np.int64, count=S)
            positions = np.asarray(q_start, dtype=np.int64)
            token_seq = np.arange(S, dtype=np.int64)
            slot_maps = []
            for g in range(ng):
                sm = []
                for tab, p in zip(tables[g], q_start):
                    page = tab[p // ps]
                    if page < 0:
                        raise StepError("a position of this step lies in a page that was given back")
                    sm.append(page * ps + p % ps)
                slot_maps.append(sm)
        else:
            token_ids = np.concatenate([np.asarray(a, dtype=np.int64) for a in toks])
            positions = np.concatenate([np.arange(a, a + n, dtype=np.int64) for a, n in zip(q_start, q_lens)])
            token_seq = np.repeat(np.arange(S, dtype=np.int64), q_lens)
            slot_maps = []
            for g in range(ng):
                parts = []
                for tab, a, n in zip(tables[g], q_start, q_lens):
                    pos = np.arange(a, a + n, dtype=np.int64)
                    pages = np.asarray(tab, dtype=np.int64)[pos // ps]
                    if pages.min() < 0:
                        raise StepError("a position of this step lies in a page that was given back")
                    parts.append(pages * ps + pos % ps)
                slot_maps.append(np.concatenate(parts))
        logit_rows: List[int] = []
        for s, en in enumerate(entries):
            base = int(cu_q[s])
            logit_rows.extend(base + int(w) for w in en.want)
        max_pages = []
        for g in range(ng):
            mp = max(len(t) for t in tables[g])
            max_pages.append(max(16, 1 << (mp - 1).bit_length()))   # powers of two: few distinct shapes for captured graphs
        tiles = [] if T == S else attention_tiles(q_lens, q_start)
        wide = [] if T == S else attention_tiles(q_lens, q_start, ATTN_TILE_WIDE)
        layout = StepLayout.make(T, S, len(logit_rows), max_pages, len(tiles) // 3, len(wide) // 3)
        i, host = self._staging(layout.total)
        self._last_layout_total = layout.total
        pack_step(layout, host.numpy(), token_ids=token_ids, positions=positions, token_seq=token_seq,
                  logit_rows=logit_rows, state_slots=slots, cu_q=cu_q, q_start=q_start, ctx_len=ctx_len,
                  slot_mappings=slot_maps, block_tables=tables, attn_tiles=tiles, attn_tiles_wide=wide)
        self._dev[:layout.total].copy_(host[:layout.total], non_blocking=True)
        self._host_events[i].record()
        self._pending_ids = pending
        # the device views of a layout are always the same tensors: keep them, refresh the host-side facts
        key = (layout.key(), self._dev.data_ptr())
        ctx = self._ctx_cache.get(key)
        if ctx is None:
            if len(self._ctx_cache) > 256:
                self._ctx_cache.clear()
            ctx = StepContext(layout, self._dev, self.ws, q_lens=q_lens, q_starts=q_start)
            self._ctx_cache[key] = ctx
        else:
            ctx.set_host_facts(q_lens, q_start)
        return ctx

    def step(self, entries: Sequence[StepEntry], commit: bool = True,
             sampled: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run one batch; returns 32-bit logits [number of wanted places, vocab] in the
        order of the entries and of each entry's ``want`` (a view that the next step
        overwrites), or None if nothing was wanted.  ``commit=False`` leaves it to the
        caller (the scheduler) to tell the cache manager that the tokens are in."""
        ctx = self.prepare_step(entries, sampled)
        if self._pending_ids:
            ops.resolve_tokens(ctx.token_ids, sampled)
        logits = self._forward(ctx)
        if commit:
            for en in entries:
                self.cache.commit(en.req, len(en.tokens))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ CUDA graphs
    def _buffer_version(self):
        """Changes whenever a scratch buffer that a captured graph may point into is replaced."""
        return (self.ws.version, ops.scratch_version)

    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """A step is about a hundred launches; issued one by one from Python they cost
        more host time than a decode step or a 2,048-token prefill takes on the GPU.  So a
        step shape that comes back (the same numbers of tokens, requests, wanted rows,
        block-table width, attention tiles and key splits: every host-side number a launch
        depends on) is captured once as a CUDA graph and replayed; a shape seen for the
        first time runs eagerly.  All graphs are dropped when a scratch buffer is replaced
        by a larger one, since a graph fixes buffer addresses."""
        if not (self.engine.use_cuda_graphs and self._graph_ok):
            with ops.stream_scope():
                return self.model.forward(ctx)
        if self._graph_version != self._buffer_version():
            self._graphs.clear()
            self._graph_seen.clear()
            self._graph_families.clear()
            self._graph_version = self._buffer_version()
        key = (ctx.layout.key(), ops.decode_splits(ctx.max_ctx_len) if ctx.decode_only else 0)
        g = self._graphs.get(key)
        if g is not None:
            g[0].replay()
            self.graph_replays += 1
            ops.launches += self.graph_kernels[key]
            return g[1]
        seen = self._graph_seen.get(key, 0)
        if len(self._graph_seen) > 4096:
            self._graph_seen.clear()
        self._graph_seen[key] = seen + 1
        # A shape that differs from a captured one only in the width of the block tables or the number of
        # key splits (a context that grew) needs no new buffers: capture it at first sight.
        family = key[0][:3] + key[0][4:]
        if seen == 0 and family not in self._graph_families:
            with ops.stream_scope():
                logits = self.model.forward(ctx)       # first time: eager, buffers get allocated
            if not self._capture_at_once:
                return logits
            # "at_once": the same step again, captured and replayed, so that even a shape that never comes back
            # is computed by a replayed graph (what the replay tests grade); a step only writes its own tokens'
            # cache slots and scratch, so running it twice changes nothing
        version = self._buffer_version()
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = ops.launches
        with torch.cuda.graph(graph):
            with ops.stream_scope():
                logits = self.model.forward(ctx)
        kernels = ops.launches - n0
        if self._buffer_version() != version:           # a buffer was allocated during capture: do not keep it
            self._graph_version = None
            with ops.stream_scope():
                return self.model.forward(ctx)
        if len(self._graphs) >= 64:
            old = next(iter(self._graphs))
            self._graphs.pop(old)
            self.graph_kernels.pop(old, None)
        self._graphs[key] = (graph, logits)
        self._graph_families.add(family)
        self.graph_kernels[key] = kernels
        ops.launches = n0 + kernels
        graph.replay()
        self.graph_replays += 1
        return logits
