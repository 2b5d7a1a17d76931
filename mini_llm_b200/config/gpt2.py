"""GPT2Config: the keys of a Hugging Face GPT-2 config.json, typed and checked.

Every value the reference keeps in include/constants.h:5-28 (layers 12, heads
12, width 768, inner 3072, vocabulary 50257, positions 1024, EOS 50256) is a
field here and is read from the file.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional

from .base import ConfigError, ModelConfig

_TANH_GELUS = ("gelu_new", "gelu_pytorch_tanh", "gelu_fast")
_ERF_GELUS = ("gelu",)

_REQUIRED = ("vocab_size", "n_positions", "n_embd", "n_layer", "n_head")


def _as_int(d, key, default=None, minimum=1):
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: missing required key {key!r}")
    if isinstance(v, bool) or not isinstance(v, int):
        if isinstance(v, float) and v == int(v):
            v = int(v)
        else:
            raise ConfigError(f"config.json: {key!r} must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {key!r} must be >= {minimum}, got {v}")
    return v


@dataclass
class GPT2Config(ModelConfig):
    vocab_size: int = 0
    n_positions: int = 0
    n_embd: int = 0
    n_layer: int = 0
    n_head: int = 0
    n_inner: int = 0                       # null in config.json means 4 * n_embd
    activation_function: str = "gelu_new"
    layer_norm_epsilon: float = 1e-5
    scale_attn_weights: bool = True
    scale_attn_by_inverse_layer_idx: bool = False
    tie_word_embeddings: bool = True
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def activation_kind(self) -> str:
        return "gelu_tanh" if self.activation_function in _TANH_GELUS else "gelu_erf"

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GPT2Config":
        missing = [k for k in _REQUIRED if d.get(k) is None]
        if missing:
            raise ConfigError(f"config.json: missing required key(s): {', '.join(missing)}")
        mt = d.get("model_type", "gpt2")
        if mt != "gpt2":
            raise ConfigError(f"config.json: model_type must be 'gpt2' for GPT2LMHeadModel, got {mt!r}")
        n_embd = _as_int(d, "n_embd")
        n_head = _as_int(d, "n_head")
        if n_embd % n_head != 0:
            raise ConfigError(f"config.json: n_embd={n_embd} is not divisible by n_head={n_head}")
        n_inner = d.get("n_inner")
        n_inner = 4 * n_embd if n_inner is None else _as_int(d, "n_inner")
        act = d.get("activation_function", "gelu_new")
        if act not in _TANH_GELUS + _ERF_GELUS:
            raise ConfigError(
                f"config.json: unknown activation_function {act!r}; known: "
                f"{', '.join(_TANH_GELUS + _ERF_GELUS)}")
        eps = d.get("layer_norm_epsilon", 1e-5)
        if not isinstance(eps, (int, float)) or isinstance(eps, bool) or not eps > 0:
            raise ConfigError(f"config.json: layer_norm_epsilon must be a positive number, got {eps!r}")
        for key in ("scale_attn_weights", "scale_attn_by_inverse_layer_idx", "tie_word_embeddings"):
            if key in d and not isinstance(d[key], bool):
                raise ConfigError(f"config.json: {key!r} must be true or false, got {d[key]!r}")
        eos = d.get("eos_token_id")
        vocab = _as_int(d, "vocab_size")
        if eos is not None:
            if isinstance(eos, bool) or not isinstance(eos, int) or not (0 <= eos < vocab):
                raise ConfigError(f"config.json: eos_token_id {eos!r} is not a token of the vocabulary")
        cfg = cls(
            vocab_size=vocab,
            n_positions=_as_int(d, "n_positions"),
            n_embd=n_embd,
            n_layer=_as_int(d, "n_layer"),
            n_head=n_head,
            n_inner=n_inner,
            activation_function=act,
            layer_norm_epsilon=float(eps),
            scale_attn_weights=bool(d.get("scale_attn_weights", True)),
            scale_attn_by_inverse_layer_idx=bool(d.get("scale_attn_by_inverse_layer_idx", False)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            eos_token_id=eos,
            torch_dtype=d.get("torch_dtype"),
        )
        cfg.architecture = "GPT2LMHeadModel"
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.pop("architecture", None)
        d["architectures"] = [self.architecture or "GPT2LMHeadModel"]
        d["model_type"] = "gpt2"
        return d
