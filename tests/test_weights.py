"""safetensors reading/writing, the loader's single error, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import mini_llm_b200 as m
from mini_llm_b200.config.base import get_architecture, load_config
from mini_llm_b200.engine.runner import Runtime
from mini_llm_b200.parts.model import Model
from mini_llm_b200.weights.loader import WeightsError, load_weights
from mini_llm_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from helpers import CONFIG_A, CONFIG_B, make_tensors, write_model


def _load(folder, dtype=torch.float32):
    cfg = load_config(folder)
    spec = get_architecture(cfg.architecture).build_spec(cfg)
    model = Model(spec)
    load_weights(model, spec, folder, Runtime(dtype=dtype, device=torch.device("cpu"), ops=None))
    return cfg, spec, model


def test_roundtrip_with_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    write_safetensors(str(tmp_path / "x.safetensors"), t.items())
    back = load_file(str(tmp_path / "x.safetensors"))
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    save_file(t, str(tmp_path / "y.safetensors"))
    with SafetensorsFile(str(tmp_path / "y.safetensors")) as f:
        assert sorted(f.names()) == ["a", "b", "c"]
        for k in t:
            assert f.shape(k) == tuple(t[k].shape) and torch.equal(f.tensor(k), t[k])


def test_broken_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))


def test_loads_conv1d_layout_and_dtypes(tmp_path):
    t = make_tensors(CONFIG_B, 3)
    d = write_model(str(tmp_path / "m"), CONFIG_B, t)
    _, _, model = _load(d, torch.bfloat16)
    att = model.layers[1].mixer
    assert att.qkv_weight.shape == (3 * 96, 96) and att.qkv_weight.dtype == torch.bfloat16
    assert torch.equal(att.qkv_weight, t["h.1.attn.c_attn.weight"].t().to(torch.bfloat16))
    assert att.qkv_bias.dtype == torch.float32 and torch.equal(att.qkv_bias, t["h.1.attn.c_attn.bias"])
    assert model.layers[0].ff.fc_weight.shape == (320, 96)
    assert model.final_norm.weight.dtype == torch.float32
    assert model.embedding.table.dtype == torch.bfloat16 and model.positions.table.shape == (256, 96)
    assert model.head.table is model.embedding.table          # tied
    _, _, m32 = _load(d, torch.float32)
    assert m32.layers[2].ff.proj_weight.dtype == torch.float32


def test_accepts_transformer_prefix_and_old_mask_buffers(tmp_path):
    t = {("transformer." + k): v for k, v in make_tensors(CONFIG_A, 1).items()}
    t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
    t["transformer.h.1.attn.masked_bias"] = torch.tensor(-1e4)
    t["lm_head.weight"] = t["transformer.wte.weight"].clone()
    d = write_model(str(tmp_path / "m"), CONFIG_A, t)
    _load(d)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    t = make_tensors(CONFIG_A, 1)
    del t["h.1.ln_2.bias"]
    del t["wpe.weight"]
    t["h.0.mlp.c_fc.weight"] = torch.zeros(64, 255)
    t["h.0.attn.c_attn.bias"] = torch.zeros(191)
    t["h.7.extra.weight"] = torch.zeros(3)
    t["stray"] = torch.zeros(1)
    d = write_model(str(tmp_path / "m"), CONFIG_A, t)
    with pytest.raises(WeightsError) as e:
        _load(d)
    err = e.value
    assert err.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert err.unexpected == ["h.7.extra.weight", "stray"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["h.0.attn.c_attn.bias", "h.0.mlp.c_fc.weight"]
    msg = str(err)
    for needle in ("h.1.ln_2.bias", "wpe.weight", "stray", "h.0.mlp.c_fc.weight", "expected [64, 256], found [64, 255]"):
        assert needle in msg


def test_untied_head_needs_its_tensor(tmp_path):
    cfg = dict(CONFIG_A, tie_word_embeddings=False)
    t = make_tensors(cfg, 1)
    d = write_model(str(tmp_path / "m"), cfg, t)
    with pytest.raises(WeightsError) as e:
        _load(d)
    assert e.value.missing == ["lm_head.weight"]
    t["lm_head.weight"] = torch.randn(512, 64)
    d = write_model(str(tmp_path / "m2"), cfg, t)
    _, _, model = _load(d)
    assert torch.equal(model.head.weight, t["lm_head.weight"])


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    d1 = m.write_random_model(CONFIG_B, 5, str(tmp_path / "a"))
    d2 = m.write_random_model(CONFIG_B, 5, str(tmp_path / "b"))
    d3 = m.write_random_model(CONFIG_B, 6, str(tmp_path / "c"))
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    f1, f2, f3 = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (d1, d2, d3))
    assert f1.names() == f2.names() and len(f1.names()) == 2 + 12 * 3 + 2
    assert all(torch.equal(f1.tensor(n), f2.tensor(n)) for n in f1.names())          # same seed, same weights
    assert not torch.equal(f1.tensor("wte.weight"), f3.tensor("wte.weight"))
    assert f1.shape("h.0.attn.c_attn.weight") == (96, 288)                          # Conv1D [in, out]
    assert torch.all(f1.tensor("h.2.ln_1.weight") == 1) and torch.all(f1.tensor("h.2.mlp.c_proj.bias") == 0)
    std = f1.tensor("h.1.mlp.c_proj.weight").std().item()
    assert abs(std - 0.02 / (2 * 3) ** 0.5) < 1e-3
    assert abs(f1.tensor("wte.weight").std().item() - 0.02) < 1e-3
    _load(d1)
    cfg = json.load(open(os.path.join(d1, "config.json")))
    assert cfg["n_inner"] == 320 and cfg["architectures"] == ["GPT2LMHeadModel"]
    d4 = m.write_random_model(CONFIG_A, 1, str(tmp_path / "d"), dtype="bfloat16")
    with SafetensorsFile(os.path.join(d4, "model.safetensors")) as f:
        assert f.dtype("wte.weight") == torch.bfloat16


def test_sharded_checkpoint_with_an_index(tmp_path):
    """model.safetensors.index.json names the shard of every tensor; loading gives the same model, and the
    single error still lists what is missing, unexpected or misshapen across the shards."""
    t = make_tensors(CONFIG_A, 5)
    whole = write_model(str(tmp_path / "whole"), CONFIG_A, t)
    d = tmp_path / "sharded"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(CONFIG_A))
    names = sorted(t)
    shards = {"model-00001-of-00002.safetensors": names[:len(names) // 2], "model-00002-of-00002.safetensors": names[len(names) // 2:]}
    for fname, ns in shards.items():
        write_safetensors(str(d / fname), [(n, t[n]) for n in ns])
    (d / "model.safetensors.index.json").write_text(json.dumps(
        {"metadata": {}, "weight_map": {n: f for f, ns in shards.items() for n in ns}}))
    _, _, a = _load(whole)
    _, _, b = _load(str(d))
    for la, lb in zip(a.layers, b.layers):
        assert torch.equal(la.mixer.qkv_weight, lb.mixer.qkv_weight) and torch.equal(la.ff.proj_weight, lb.ff.proj_weight)
    assert torch.equal(a.embedding.table, b.embedding.table)
    # a shard that lacks a tensor the index promises
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), [(n, t[n]) for n in shards["model-00002-of-00002.safetensors"][1:]])
    with pytest.raises(SafetensorsError, match="is not in"):
        _load(str(d))
    # an extra tensor in a shard and a wrong shape elsewhere: one error for both
    extra = [(n, t[n]) for n in shards["model-00002-of-00002.safetensors"]] + [("stray.weight", torch.zeros(2))]
    write_safetensors(str(d / "model-00002-of-00002.safetensors"), extra)
    first = shards["model-00001-of-00002.safetensors"]
    write_safetensors(str(d / "model-00001-of-00002.safetensors"), [(n, t[n] if n != first[0] else torch.zeros(3, 3)) for n in first])
    with pytest.raises(WeightsError) as e:
        _load(str(d))
    assert "stray.weight" in e.value.unexpected and e.value.wrong_shape and e.value.wrong_shape[0][0] == first[0]
