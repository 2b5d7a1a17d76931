"""Loading a model's parameters from model.safetensors (or its shards) by tensor name.

Every part declares its parameters (``param_specs``); the model description
says which checkpoint tensor each one is (``WeightRef``).  All problems are
collected and reported in ONE error: tensors that are missing, tensors that
nothing asked for, and tensors whose shape does not fit the configuration.
The reference stops at the first missing or short file with exit(1)
(src/model/gpt2_model.cu:35-55).

Kept dtypes: matrices and embedding tables in the engine dtype (bfloat16 when
serving; float32 on the 32-bit path), norm weights and biases in float32 (a
32-bit tensor is never narrowed for them), integer tables as int32.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List

import torch

from ..parts.spec import ModelSpec
from .safetensors_io import Checkpoint


class WeightsError(ValueError):
    """model.safetensors does not fit the model; lists everything that is wrong."""

    def __init__(self, path, missing, unexpected, wrong_shape, other=()):
        self.path = path
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"{path}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(g)}" for n, e, g in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def checkpoint_shape(shape, ref):
    """Shape of a parameter as the checkpoint stores it."""
    return tuple(reversed(shape)) if ref.transpose and len(shape) == 2 else tuple(shape)


def target_dtype(role: str, engine_dtype: torch.dtype) -> torch.dtype:
    if role in ("matrix", "table"):
        return engine_dtype
    if role == "int":
        return torch.int32
    return torch.float32


def load_weights(model, spec: ModelSpec, model_dir: str, rt) -> None:
    """Read, check, convert, upload and bind every parameter of ``model``."""
    sf = Checkpoint(model_dir)       # model.safetensors, or the shards named by model.safetensors.index.json
    path = sf.path
    try:
        names = set(sf.names())
        used = set()
        missing: List[str] = []
        wrong = []
        other: List[str] = []
        plan = []     # (part, local, found_name, ref, pspec)
        for label, pspec_part in spec.all_part_specs():
            part = model.part(label)
            wanted = part.param_specs()
            for local in wanted:
                if local not in pspec_part.weights:
                    other.append(f"{label}: the model description names no tensor for parameter {local!r}")
            for local, ref in pspec_part.weights.items():
                if local not in wanted:
                    other.append(f"{label}: the description gives a tensor for {local!r}, which the part does not have")
                    continue
                found = next((n for n in ref.names if n in names), None)
                if found is None:
                    missing.append(ref.canonical)
                    continue
                used.add(found)
                exp = checkpoint_shape(wanted[local].shape, ref)
                got = sf.shape(found)
                if tuple(got) != tuple(exp):
                    wrong.append((found, exp, got))
                    continue
                if not (sf.dtype(found).is_floating_point or wanted[local].role == "int"):
                    other.append(f"{found}: dtype {sf.dtype(found)} cannot feed a {wanted[local].role} parameter")
                    continue
                plan.append((part, local, found, ref, wanted[local]))
        ignore = [re.compile(p) for p in spec.ignored_tensors]
        unexpected = sorted(n for n in names - used if not any(r.search(n) for r in ignore))
        if missing or unexpected or wrong or other:
            raise WeightsError(path, sorted(missing), unexpected, wrong, other)
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        parts = {}
        for part, local, found, ref, ps in plan:
            t = sf.tensor(found)
            if ref.transpose and t.dim() == 2:
                t = t.t()
            t = t.to(target_dtype(ps.role, rt.dtype)).contiguous()
            per_part.setdefault(id(part), {})[local] = t.to(rt.device)
            parts[id(part)] = part
    finally:
        sf.close()
    for label, _ in spec.all_part_specs():
        part = model.part(label)
        part.bind(per_part.get(id(part), {}), rt)
    model.finish_binding(rt)
