"""GPT-2 (``GPT2LMHeadModel``): configuration -> model description.

A pre-LayerNorm decoder with learned absolute token and position embeddings,
a fused c_attn projection, multi-head causal attention, a GELU MLP, a final
LayerNorm and a head tied to wte: the model the reference runs in
src/model/gpt2_model.cu.  Tensor names are the checkpoint's
(scripts/export_weights.py:34-66 lists them; old checkpoints prefix them with
"transformer."); Conv1D matrices are stored [in, out] (:48-52) and are
transposed once at load so every product reads both operands along the
contraction dimension.
"""
from __future__ import annotations

import math

from ..config.base import register_architecture
from ..config.gpt2 import GPT2Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, WeightRef


def _names(n):
    return (n, "transformer." + n)


def build_gpt2_spec(cfg: GPT2Config) -> ModelSpec:
    D, H, dh = cfg.n_embd, cfg.n_head, cfg.head_dim
    std = 0.02
    proj_std = 0.02 / math.sqrt(2 * cfg.n_layer)
    ones, zeros = ("ones",), ("zeros",)

    def norm(prefix):
        return PartSpec("layernorm", dict(hidden_size=D, eps=cfg.layer_norm_epsilon),
                        {"weight": WeightRef(_names(prefix + ".weight"), init=ones),
                         "bias": WeightRef(_names(prefix + ".bias"), init=zeros)})

    layers = []
    for l in range(cfg.n_layer):
        p = f"h.{l}."
        scale = 1.0 / math.sqrt(dh) if cfg.scale_attn_weights else 1.0
        if cfg.scale_attn_by_inverse_layer_idx:
            scale /= float(l + 1)
        mixer = PartSpec(
            "attention",
            dict(hidden_size=D, num_heads=H, num_kv_heads=H, head_dim=dh, scale=scale, window=None, bias=True),
            {"qkv_weight": WeightRef(_names(p + "attn.c_attn.weight"), transpose=True, init=("normal", std)),
             "qkv_bias": WeightRef(_names(p + "attn.c_attn.bias"), init=zeros),
             "out_weight": WeightRef(_names(p + "attn.c_proj.weight"), transpose=True, init=("normal", proj_std)),
             "out_bias": WeightRef(_names(p + "attn.c_proj.bias"), init=zeros)})
        ff = PartSpec(
            "mlp",
            dict(hidden_size=D, inner_size=cfg.n_inner, activation=cfg.activation_kind, bias=True),
            {"fc_weight": WeightRef(_names(p + "mlp.c_fc.weight"), transpose=True, init=("normal", std)),
             "fc_bias": WeightRef(_names(p + "mlp.c_fc.bias"), init=zeros),
             "proj_weight": WeightRef(_names(p + "mlp.c_proj.weight"), transpose=True, init=("normal", proj_std)),
             "proj_bias": WeightRef(_names(p + "mlp.c_proj.bias"), init=zeros)})
        layers.append(LayerSpec(mixer=mixer, ff=ff, mixer_norm=norm(p + "ln_1"), ff_norm=norm(p + "ln_2"),
                                arrangement="pre_norm"))

    embedding = PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab_size),
                         {"table": WeightRef(_names("wte.weight"), init=("normal", std))})
    positions = PartSpec("learned", dict(hidden_size=D, max_positions=cfg.n_positions),
                         {"table": WeightRef(_names("wpe.weight"), init=("normal", std))})
    if cfg.tie_word_embeddings:
        head = PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab_size))
    else:
        head = PartSpec("linear", dict(hidden_size=D, vocab_size=cfg.vocab_size),
                        {"weight": WeightRef(("lm_head.weight",), init=("normal", std))})
    ignored = [r"^(transformer\.)?h\.\d+\.attn\.(bias|masked_bias)$"]   # causal-mask buffers of old checkpoints
    if cfg.tie_word_embeddings:
        ignored.append(r"^lm_head\.weight$")
    return ModelSpec(hidden_size=D, vocab_size=cfg.vocab_size, embedding=embedding, positions=positions,
                     layers=layers, final_norm=norm("ln_f"), head=head, max_positions=cfg.n_positions,
                     eos_token_id=cfg.eos_token_id, ignored_tensors=ignored)


register_architecture("GPT2LMHeadModel", GPT2Config, build_gpt2_spec, replace=True)
