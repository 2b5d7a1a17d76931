"""Typed configuration and the architecture registry.

The reference engine fixes every model size at compile time
(include/constants.h:5-28).  Here every size comes from the model folder's
``config.json``; the ``architectures`` entry of that file selects, through one
registry, the configuration class and the function that turns a configuration
into a model description (``ModelSpec``).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


@dataclass
class ModelConfig:
    """Base class of every architecture's typed configuration."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":  # pragma: no cover
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:  # pragma: no cover
        raise NotImplementedError


@dataclass
class EngineConfig:
    """Sizes of the engine around the model (none of them is a model size).

    The reference has these as constants too: page ("block") size 16 and 4096
    pages (include/constants.h:16-17), at most 16 requests per model call
    (include/constants.h:26).
    """

    dtype: str = "bfloat16"            # "bfloat16" | "float32"
    page_size: int = 16                # tokens per cache page
    num_pages: Optional[int] = None    # pages per cache group (None: from max_tokens)
    max_tokens: Optional[int] = None   # tokens the cache pool must hold (None: from memory)
    max_num_seqs: int = 64             # live requests (state slots, block-table rows)
    max_num_batched_tokens: int = 2048  # token budget of one step
    prefill_chunk: int = 2048          # largest portion of one prompt in one step
    admission: str = "lazy"            # "lazy" | "reserve"
    memory_fraction: float = 0.5       # of free device memory, when sizes are not given
    use_cuda_graphs: bool = True
    graph_capture: str = "on_return"   # "on_return": a step shape is captured when it comes back; "at_once": at first sight
    use_pdl: bool = True               # programmatic dependent launch between the kernels of a step
    async_scheduling: bool = True      # while only decodes run, launch a step before the last one's tokens are read
    device: str = "cuda:0"

    def __post_init__(self):
        if self.dtype in ("bf16",):
            self.dtype = "bfloat16"
        if self.dtype in ("fp32", "f32"):
            self.dtype = "float32"
        if self.dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"dtype must be bfloat16 or float32, got {self.dtype!r}")
        if self.page_size <= 0:
            raise ConfigError(f"page_size must be positive, got {self.page_size}")
        if self.max_num_seqs <= 0:
            raise ConfigError("max_num_seqs must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ConfigError("max_num_batched_tokens must be positive")
        if self.prefill_chunk <= 0:
            raise ConfigError("prefill_chunk must be positive")
        if self.graph_capture not in ("on_return", "at_once"):
            raise ConfigError(f"graph_capture must be 'on_return' or 'at_once', got {self.graph_capture!r}")
        if self.admission not in ("lazy", "reserve"):
            raise ConfigError(f"admission must be 'lazy' or 'reserve', got {self.admission!r}")


@dataclass
class Architecture:
    """One registry entry: how an ``architectures`` name becomes a model."""

    name: str
    config_cls: type
    build_spec: Callable[[Any], Any]          # config -> parts.spec.ModelSpec
    extra: Dict[str, Any] = field(default_factory=dict)


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable[[Any], Any],
                          *, replace: bool = False) -> Architecture:
    """Register an architecture under the name config.json gives it."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    arch = Architecture(name=name, config_cls=config_cls, build_spec=build_spec)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
        raise ConfigError(f"unknown architecture {name!r}; registered: {known}")
    return _ARCHITECTURES[name]


def registered_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    """Pick the architecture named by ``architectures`` and parse its keys."""
    archs = d.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list")
    last_err: Optional[Exception] = None
    for name in archs:
        if name in _ARCHITECTURES:
            arch = _ARCHITECTURES[name]
            cfg = arch.config_cls.from_dict(d)
            cfg.architecture = name
            return cfg
        last_err = ConfigError(f"unknown architecture {name!r}")
    known = ", ".join(sorted(_ARCHITECTURES)) or "(none)"
    raise ConfigError(f"none of the architectures {list(archs)} is registered; registered: {known}") from last_err


def load_config(model_dir: str) -> ModelConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return config_from_dict(d)
