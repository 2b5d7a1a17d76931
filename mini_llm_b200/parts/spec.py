"""The description of a model as data.

An architecture's ``build_spec(config)`` returns a ``ModelSpec``: which part
(by registry key) stands where, with which constants and which checkpoint
tensors, layer by layer, and in which order the layers run.  Nothing in here
executes; ``parts.model.Model`` builds the parts from it.

The reference has no such level: GPT2Model hard-wires twelve identical blocks
(src/model/gpt2_model.cu:271-365, 402-406).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple


@dataclass
class WeightRef:
    """Where one parameter of a part comes from in the checkpoint.

    ``names``: accepted tensor names, the first is canonical (the one written by
    the random-weights mode).  ``transpose``: the checkpoint stores the matrix
    [in, out] (GPT-2's Conv1D, scripts/export_weights.py:48-52) while parts keep
    matrices [out, in].  ``init``: ("normal", std) | ("ones",) | ("zeros",) for
    the random-weights mode.  ``shared_with``: canonical name of a tensor that
    this parameter aliases (a tied head), so it is neither stored nor missed.
    """

    names: Sequence[str]
    transpose: bool = False
    init: Tuple = ("normal", 0.02)
    shared_with: Optional[str] = None

    @property
    def canonical(self) -> str:
        return self.names[0]


@dataclass
class PartSpec:
    """One part: registry key, constructor constants, checkpoint tensors."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, WeightRef] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One block: a mixer and a feed-forward, each behind its norm.

    ``arrangement`` names how they are wired (registry ``ARRANGEMENTS``), e.g.
    "pre_norm": x += mixer(norm(x)); x += ff(norm(x)).
    """

    mixer: PartSpec
    ff: PartSpec
    mixer_norm: PartSpec
    ff_norm: PartSpec
    arrangement: str = "pre_norm"


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``cache_of``: the layer whose cache (pages or state)
    this run uses; when it differs from ``layer`` the run only reads that cache
    and writes nothing to it."""

    layer: int
    cache_of: Optional[int] = None

    def __post_init__(self):
        if self.cache_of is None:
            self.cache_of = self.layer


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    positions: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    head: PartSpec
    schedule: Optional[List[ScheduleEntry]] = None
    max_positions: Optional[int] = None      # None: the position encoding sets no limit
    eos_token_id: Optional[int] = None
    ignored_tensors: List[str] = field(default_factory=list)   # regexes of checkpoint tensors to skip

    def __post_init__(self):
        if self.schedule is None:
            self.schedule = [ScheduleEntry(i) for i in range(len(self.layers))]
        n = len(self.layers)
        for e in self.schedule:
            if not (0 <= e.layer < n) or not (0 <= e.cache_of < n):
                raise ValueError(f"schedule entry {e} names a layer outside 0..{n - 1}")

    def all_part_specs(self):
        """(label, PartSpec) of every part, in a fixed order."""
        yield "embedding", self.embedding
        yield "positions", self.positions
        for i, l in enumerate(self.layers):
            yield f"layers.{i}.mixer_norm", l.mixer_norm
            yield f"layers.{i}.mixer", l.mixer
            yield f"layers.{i}.ff_norm", l.ff_norm
            yield f"layers.{i}.ff", l.ff
        yield "final_norm", self.final_norm
        yield "head", self.head
