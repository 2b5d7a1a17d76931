"""The writer of the reference's weight format (one raw float32 file per tensor): names, sizes and
layout against src/model/gpt2_model.cu:115-173, and the refusal of models the reference cannot run."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import CONFIG_A, make_model, make_tensors
from mini_llm_b200.weights.reference_bins import REFERENCE_SIZES, reference_bin_files, write_reference_bins


def test_files_are_the_ones_the_reference_opens():
    files = reference_bin_files(12, 768, 3072, 50257, 1024)
    names = [f for f, _, _ in files]
    assert len(names) == 2 + 12 * 12 + 2 and len(set(names)) == len(names)
    assert names[:2] == ["wte.bin", "wpe.bin"] and names[-2:] == ["ln_f_w.bin", "ln_f_b.bin"]
    per_layer = ["ln1_w", "ln1_b", "qkv_w", "qkv_b", "out_w", "out_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b"]
    assert names[2:14] == [f"{p}_0.bin" for p in per_layer]
    shapes = {f: s for f, _, s in files}
    # element counts as load_weights asks for them
    assert np.prod(shapes["qkv_w_3.bin"]) == 3 * 768 * 768 and shapes["qkv_w_3.bin"] == (768, 2304)
    assert shapes["fc1_w_11.bin"] == (768, 3072) and shapes["fc2_w_11.bin"] == (3072, 768)
    assert shapes["wte.bin"] == (50257, 768) and shapes["wpe.bin"] == (1024, 768)
    total = sum(int(np.prod(s)) for s in shapes.values())
    assert total == 124_439_808                        # GPT-2 small's parameter count


def test_layout_is_the_checkpoints_own(tmp_path):
    d = make_model(str(tmp_path / "m"), "A", seed=5)
    out = str(tmp_path / "bins")
    written = write_reference_bins(d, out, require_reference_sizes=False)
    t = make_tensors(CONFIG_A, 5)
    D, F = CONFIG_A["n_embd"], CONFIG_A["n_inner"]
    assert written["qkv_w_1.bin"] == D * 3 * D and written["fc1_b_0.bin"] == F
    # Conv1D matrices stay [in, out], row-major, little-endian float32: element (i, o) at i * out + o
    w = np.fromfile(os.path.join(out, "qkv_w_1.bin"), dtype="<f4").reshape(D, 3 * D)
    assert np.array_equal(w, t["h.1.attn.c_attn.weight"].numpy())
    w = np.fromfile(os.path.join(out, "fc2_w_0.bin"), dtype="<f4").reshape(F, D)
    assert np.array_equal(w, t["h.0.mlp.c_proj.weight"].numpy())
    assert np.array_equal(np.fromfile(os.path.join(out, "wte.bin"), dtype="<f4"), t["wte.weight"].numpy().ravel())
    assert np.array_equal(np.fromfile(os.path.join(out, "ln_f_b.bin"), dtype="<f4"), t["ln_f.bias"].numpy())
    for f, n in written.items():
        assert os.path.getsize(os.path.join(out, f)) == 4 * n


def test_bfloat16_checkpoints_are_widened(tmp_path):
    d = make_model(str(tmp_path / "m"), "A", seed=6, dtype=torch.bfloat16)
    out = str(tmp_path / "bins")
    write_reference_bins(d, out, require_reference_sizes=False)
    t = make_tensors(CONFIG_A, 6)
    got = np.fromfile(os.path.join(out, "wpe.bin"), dtype="<f4")
    assert np.array_equal(got, t["wpe.weight"].to(torch.bfloat16).float().numpy().ravel())


def test_other_sizes_are_refused(tmp_path):
    d = make_model(str(tmp_path / "m"), "A", seed=1)
    with pytest.raises(ValueError, match="GPT-2 small only"):
        write_reference_bins(d, str(tmp_path / "bins"))
    assert REFERENCE_SIZES["vocab_size"] == 50257


def test_a_missing_tensor_is_named(tmp_path):
    from helpers import write_model
    t = make_tensors(CONFIG_A, 2)
    del t["h.1.mlp.c_fc.bias"]
    d = write_model(str(tmp_path / "m"), CONFIG_A, t)
    with pytest.raises(ValueError, match="h.1.mlp.c_fc.bias"):
        write_reference_bins(d, str(tmp_path / "bins"), require_reference_sizes=False)
