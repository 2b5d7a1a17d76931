"""Random-weights mode: write a model folder from a configuration and a seed.

The folder holds config.json and model.safetensors with the architecture's own
tensor names and layouts, so it loads like any checkpoint.  Rules come from
the model description's ``WeightRef.init``: N(0, std) matrices and tables,
ones / zeros for norm weights and biases.  Values are drawn on the CPU in
32-bit from one seeded generator, tensor by tensor in the description's order,
then stored in ``dtype``.  (The reference has no such mode: it needs the real
checkpoint exported by scripts/export_weights.py.)
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Union

import torch

from ..config.base import ModelConfig, config_from_dict, get_architecture
from .loader import checkpoint_shape
from .safetensors_io import write_safetensors

_STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def random_tensors(spec, model, seed: int, dtype: torch.dtype = torch.float32):
    """Yield (canonical name, tensor as the checkpoint stores it)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    for label, pspec in spec.all_part_specs():
        part = model.part(label)
        wanted = part.param_specs()
        for local, ref in pspec.weights.items():
            shape = checkpoint_shape(wanted[local].shape, ref)
            kind = ref.init[0]
            if kind == "normal":
                t = torch.empty(shape, dtype=torch.float32).normal_(0.0, float(ref.init[1]), generator=gen)
            elif kind == "ones":
                t = torch.ones(shape, dtype=torch.float32)
            elif kind == "zeros":
                t = torch.zeros(shape, dtype=torch.float32)
            else:
                raise ValueError(f"{ref.canonical}: unknown init rule {ref.init!r}")
            if wanted[local].role == "int":
                t = t.to(torch.int32)
            else:
                t = t.to(dtype)
            yield ref.canonical, t


def write_random_model(config: Union[Dict[str, Any], ModelConfig], seed: int, out_dir: str,
                       dtype: str = "float32") -> str:
    """Create ``out_dir`` with config.json and model.safetensors; returns out_dir."""
    from ..parts.model import Model

    if dtype not in _STORE:
        raise ValueError(f"dtype must be one of {sorted(_STORE)}, got {dtype!r}")
    cfg_dict = config.to_dict() if isinstance(config, ModelConfig) else dict(config)
    cfg = config_from_dict(cfg_dict)
    arch = get_architecture(cfg.architecture)
    spec = arch.build_spec(cfg)
    model = Model(spec)
    os.makedirs(out_dir, exist_ok=True)
    out_cfg = dict(cfg_dict)
    out_cfg["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out_cfg, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"),
                      random_tensors(spec, model, seed, _STORE[dtype]),
                      metadata={"format": "pt", "seed": seed})
    return out_dir
