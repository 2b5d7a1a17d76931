"""Sampling parameters and the per-token uniform numbers.

The reference picks the argmax only (src/kernels/argmax.cu; README.md "Current
Limitations" lists temperature sampling as not implemented) and stops at
max_new_tokens (default 8, include/constants.h:14; include/runtime/request.h:72-78)
or at the EOS id (src/model/gpt2_model.cu:448).  Temperature sampling is added
here: an inverse-CDF draw with a uniform number that depends on (seed, request,
index of the generated token) only, never on the batch the request sits in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional

DEFAULT_MAX_NEW_TOKENS = 8      # include/constants.h:14


@dataclass
class SamplingParams:
    temperature: float = 0.0            # 0: greedy (argmax, lowest id among equals)
    seed: int = 0
    max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS
    ignore_eos: bool = False

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")


_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return z ^ (z >> 31)


def _key_of(request_id: Hashable) -> int:
    if isinstance(request_id, int):
        return request_id & _MASK
    h = 0xCBF29CE484222325
    for b in str(request_id).encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return h


def uniform_for(seed: int, request_id: Hashable, index: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its arguments."""
    x = _splitmix64(seed & _MASK)
    x = _splitmix64(x ^ _key_of(request_id))
    x = _splitmix64(x ^ (index & _MASK))
    return (x >> 40) / float(1 << 24)
