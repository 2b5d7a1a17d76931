"""Configuration parsing and the architecture registry (no GPU)."""
import json
import os

import pytest

import mini_llm_b200 as m
from mini_llm_b200.config.base import ConfigError, EngineConfig, config_from_dict, get_architecture, load_config
from mini_llm_b200.config.gpt2 import GPT2Config
from helpers import CONFIG_A, CONFIG_B


def test_registry_maps_name_to_model():
    assert "GPT2LMHeadModel" in m.registered_architectures()
    arch = get_architecture("GPT2LMHeadModel")
    assert arch.config_cls is GPT2Config


def test_every_key_is_read_from_the_file():
    a = config_from_dict(CONFIG_A)
    b = config_from_dict(CONFIG_B)
    assert (a.n_layer, a.n_embd, a.n_head, a.head_dim, a.n_inner, a.vocab_size, a.n_positions) == (2, 64, 4, 16, 256, 512, 128)
    assert (b.n_layer, b.n_embd, b.n_head, b.head_dim, b.n_inner, b.vocab_size, b.n_positions) == (3, 96, 3, 32, 320, 1000, 256)
    assert a.layer_norm_epsilon == 1e-5 and b.layer_norm_epsilon == 1e-6
    assert a.activation_kind == "gelu_tanh" and b.activation_kind == "gelu_erf"
    assert not a.scale_attn_by_inverse_layer_idx and b.scale_attn_by_inverse_layer_idx
    assert a.eos_token_id == 511 and b.eos_token_id == 999


def test_defaults():
    d = dict(architectures=["GPT2LMHeadModel"], n_layer=1, n_embd=32, n_head=2, vocab_size=10, n_positions=8)
    c = config_from_dict(d)
    assert c.n_inner == 128 and c.activation_function == "gelu_new" and c.layer_norm_epsilon == 1e-5
    assert c.tie_word_embeddings and c.scale_attn_weights and c.eos_token_id is None


@pytest.mark.parametrize("change,needle", [
    (dict(architectures=["NoSuchModel"]), "NoSuchModel"),
    (dict(architectures=None), "architectures"),
    (dict(n_head=5), "divisible"),
    (dict(activation_function="swish"), "activation_function"),
    (dict(n_layer=None), "n_layer"),
    (dict(n_embd="64"), "integer"),
    (dict(layer_norm_epsilon=0), "layer_norm_epsilon"),
    (dict(eos_token_id=512), "eos_token_id"),
    (dict(model_type="llama"), "model_type"),
    (dict(tie_word_embeddings="yes"), "tie_word_embeddings"),
])
def test_errors(change, needle):
    d = dict(CONFIG_A)
    d.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert needle in str(e.value)


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(CONFIG_B))
    assert load_config(str(tmp_path)).n_embd == 96


def test_spec_carries_the_constants_per_layer():
    b = config_from_dict(CONFIG_B)
    spec = get_architecture(b.architecture).build_spec(b)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    scales = [l.mixer.params["scale"] for l in spec.layers]
    base = 32 ** -0.5
    assert scales == pytest.approx([base, base / 2, base / 3])
    assert all(l.mixer_norm.params["eps"] == 1e-6 for l in spec.layers)
    assert spec.layers[0].ff.params["inner_size"] == 320 and spec.layers[0].ff.params["activation"] == "gelu_erf"
    assert spec.positions.params["max_positions"] == 256 and spec.max_positions == 256


def test_engine_config_checks():
    assert EngineConfig(dtype="bf16").dtype == "bfloat16"
    for bad in (dict(dtype="fp8"), dict(page_size=0), dict(admission="greedy"), dict(max_num_seqs=0)):
        with pytest.raises(ConfigError):
            EngineConfig(**bad)


def test_a_head_size_without_a_kernel_is_refused_at_construction(tmp_path):
    """n_embd=100 over 5 heads is a valid GPT-2 configuration but gives heads of 20, which no attention kernel
    takes: the runner refuses it when it is built (before weights, pool or device), naming the limit once."""
    import json
    import pytest
    from mini_llm_b200.config.base import ConfigError, EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner

    cfg = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=100, n_head=5, vocab_size=50,
               n_positions=32)
    (tmp_path / "config.json").write_text(json.dumps(cfg))          # no weights: it must not get that far
    with pytest.raises(ConfigError) as e:
        ModelRunner(str(tmp_path), EngineConfig(dtype="float32"))
    assert "head size 20" in str(e.value) and str(e.value).count("head size 20") == 1
    # the parts are asked: heads of 48 (a multiple of 16) pass this check
    from mini_llm_b200.config.base import config_from_dict, get_architecture
    from mini_llm_b200.parts.model import Model
    ok = config_from_dict(dict(cfg, n_embd=96, n_head=2))
    assert Model(get_architecture(ok.architecture).build_spec(ok)).kernel_limits("bfloat16") == []
