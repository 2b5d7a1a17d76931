"""Turns a step's logits into next tokens on the device (csrc/sampling.cu)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from .. import ops
from .params import SamplingParams, uniform_for


class Sampler:
    """``launch`` puts the sampling kernel and the copy of its result to pinned host memory on
    the stream and returns a ticket; ``fetch`` waits for that copy and returns the tokens.
    Two sets of host buffers alternate, so one step's tokens can still be on their way
    while the next step is launched.  The device buffer ``dev_out`` always holds the tokens
    of the last launch: a following step may read its input tokens from there."""

    def __init__(self, device, max_rows: int = 64):
        self.device = device
        self._cap = 0
        self._turn = 0
        self._events = [None, None]
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self._cap:
            return
        for ev in self._events:
            if ev is not None:
                ev.synchronize()
        cap = max(n, 2 * self._cap, 64)
        self._cap = cap
        self.host_f = [torch.empty((2, cap), dtype=torch.float32, pin_memory=True) for _ in range(2)]
        self.dev_f = torch.empty((2, cap), dtype=torch.float32, device=self.device)
        self.dev_out = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self.host_out = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(2)]

    def launch(self, logits: torch.Tensor, requests: Sequence) -> Tuple[int, int]:
        """One token per row of ``logits``; ``requests[r]`` has .params, .request_id and
        .num_generated (the index of the token being drawn)."""
        R = logits.shape[0]
        if R != len(requests):
            raise ValueError("one request per row of logits")
        self._grow(R)
        i = self._turn
        self._turn ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()          # the copies that last used these host buffers are done
        else:
            self._events[i] = torch.cuda.Event()
        greedy = all(r.params.temperature == 0 for r in requests)
        if greedy:
            ops.argmax(logits, self.dev_out[:R])
        else:
            hf = self.host_f[i]
            for j, r in enumerate(requests):
                hf[0, j] = r.params.temperature
                hf[1, j] = uniform_for(r.params.seed, r.request_id, r.num_generated) if r.params.temperature > 0 else 0.0
            self.dev_f[:, :R].copy_(hf[:, :R], non_blocking=True)
            ops.sample(logits, self.dev_f[0, :R], self.dev_f[1, :R], self.dev_out[:R])
        self.host_out[i][:R].copy_(self.dev_out[:R], non_blocking=True)
        self._events[i].record()
        return i, R

    def fetch(self, ticket: Tuple[int, int]) -> List[int]:
        i, R = ticket
        self._events[i].synchronize()
        ops.raise_if_kernel_gave_up()       # the host has waited for the step: a kernel that gave up has said so by now
        return self.host_out[i][:R].tolist()

    def sample(self, logits: torch.Tensor, requests: Sequence) -> List[int]:
        return self.fetch(self.launch(logits, requests))
