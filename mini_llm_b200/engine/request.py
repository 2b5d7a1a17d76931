"""Requests and responses, with the reference's names
(include/runtime/request.h:16-79, include/runtime/response.h:6-17)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Hashable, List, Optional

import numpy as np

from ..sampling.params import SamplingParams


class RequestState(enum.Enum):
    WaitingPrefill = "waiting_prefill"
    DeferredPrefillKV = "deferred_prefill_kv"
    PrefillRunning = "prefill_running"
    DecodeReady = "decode_ready"
    DeferredDecodeKV = "deferred_decode_kv"
    DecodeRunning = "decode_running"
    Finished = "finished"
    Aborted = "aborted"


@dataclass
class Request:
    request_id: Hashable
    tokens: List[int]                       # prompt followed by generated tokens
    params: SamplingParams = field(default_factory=SamplingParams)
    prompts_len: int = 0                    # length of the original prompt
    state: RequestState = RequestState.WaitingPrefill
    num_computed: int = 0                   # tokens whose keys/values are in the cache
    num_preemptions: int = 0
    arrival: int = 0
    ended_at: Optional[int] = None          # index of the end-of-sequence token, once one was sampled

    def __post_init__(self):
        self.tokens = [int(t) for t in self.tokens]
        if not self.prompts_len:
            self.prompts_len = len(self.tokens)
        self._array = np.asarray(self.tokens, dtype=np.int32)      # the tokens known at admission, for prompt portions

    def portion(self, start: int, stop: int):
        """tokens[start:stop] as an int32 array: a view of an array made once, so that cutting a prompt into portions
        costs no conversion per step (a list of a thousand Python ints takes longer to convert than the step's other
        host work together).  After a preemption the array is rebuilt from the list, which has grown by then."""
        if stop > self._array.shape[0]:
            self._array = np.asarray(self.tokens[:stop] if stop == len(self.tokens) else self.tokens, dtype=np.int32)
        return self._array[start:stop]

    @property
    def max_new_tokens(self) -> int:
        return self.params.max_new_tokens

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.prompts_len

    def generated_tokens(self) -> List[int]:
        return self.tokens[self.prompts_len:]

    def isfinish(self) -> bool:
        return self.num_generated >= self.max_new_tokens


@dataclass
class Response:
    request_id: Hashable
    token: int
    finished: bool = False
