"""Turns a step's logits into next tokens on the device (csrc/sampling.cu)."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import ops
from .params import SamplingParams, uniform_for


class Sampler:
    def __init__(self, device, max_rows: int = 64):
        self.device = device
        self._cap = 0
        self._grow(max_rows)

    def _grow(self, n: int) -> None:
        if n <= self._cap:
            return
        cap = max(n, 2 * self._cap, 64)
        self._cap = cap
        self.host_f = torch.empty((2, cap), dtype=torch.float32, pin_memory=True)
        self.dev_f = torch.empty((2, cap), dtype=torch.float32, device=self.device)
        self.dev_out = torch.empty(cap, dtype=torch.int32, device=self.device)
        self.host_out = torch.empty(cap, dtype=torch.int32, pin_memory=True)

    def sample(self, logits: torch.Tensor, requests: Sequence) -> List[int]:
        """One token per row of ``logits``; ``requests[r]`` has .params, .request_id and
        .num_generated (the index of the token being drawn)."""
        R = logits.shape[0]
        if R != len(requests):
            raise ValueError("one request per row of logits")
        self._grow(R)
        greedy = all(r.params.temperature == 0 for r in requests)
        if greedy:
            ops.argmax(logits, self.dev_out[:R])
        else:
            hf = self.host_f
            for i, r in enumerate(requests):
                hf[0, i] = r.params.temperature
                hf[1, i] = uniform_for(r.params.seed, r.request_id, r.num_generated) if r.params.temperature > 0 else 0.0
            self.dev_f[:, :R].copy_(hf[:, :R], non_blocking=True)
            ops.sample(logits, self.dev_f[0, :R], self.dev_f[1, :R], self.dev_out[:R])
        self.host_out[:R].copy_(self.dev_out[:R], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.host_out[:R].tolist()
