"""Write a GPT-2 model folder out in the reference's own weight format.

taejuk/mini-llm reads one raw little-endian float32 file per tensor from a folder fixed at
compile time (src/model/gpt2_model.cu:32-70 ``load_bin``, :115-173 ``load_weights``):

    wte.bin [V, D]   wpe.bin [P, D]   ln_f_w.bin  ln_f_b.bin [D]
    per layer l:  ln1_w_l  ln1_b_l  ln2_w_l  ln2_b_l [D]
                  qkv_w_l [D, 3D]   qkv_b_l [3D]     out_w_l [D, D]   out_b_l [D]
                  fc1_w_l [D, F]    fc1_b_l [F]      fc2_w_l [F, D]   fc2_b_l [D]

The Conv1D matrices stay [in, out] exactly as the checkpoint stores them
(scripts/export_weights.py:48-52 "Do NOT transpose"); nothing is renamed beyond the file
names, nothing is split.  With this the unmodified reference can be run on the same seeded
random weights as this engine (its sizes are compile-time constants, include/constants.h:5-10,
so only a model of exactly those sizes can be written).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Tuple

import torch

from .safetensors_io import Checkpoint

# the sizes the reference is compiled for (include/constants.h:5-10, 25)
REFERENCE_SIZES = dict(n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024)


def reference_bin_files(n_layer: int, D: int, F: int, V: int, P: int) -> List[Tuple[str, str, Tuple[int, ...]]]:
    """(file name, checkpoint tensor name, shape) in the order the reference loads them."""
    files = [("wte.bin", "wte.weight", (V, D)), ("wpe.bin", "wpe.weight", (P, D))]
    for l in range(n_layer):
        h = f"h.{l}."
        files += [
            (f"ln1_w_{l}.bin", h + "ln_1.weight", (D,)), (f"ln1_b_{l}.bin", h + "ln_1.bias", (D,)),
            (f"qkv_w_{l}.bin", h + "attn.c_attn.weight", (D, 3 * D)), (f"qkv_b_{l}.bin", h + "attn.c_attn.bias", (3 * D,)),
            (f"out_w_{l}.bin", h + "attn.c_proj.weight", (D, D)), (f"out_b_{l}.bin", h + "attn.c_proj.bias", (D,)),
            (f"ln2_w_{l}.bin", h + "ln_2.weight", (D,)), (f"ln2_b_{l}.bin", h + "ln_2.bias", (D,)),
            (f"fc1_w_{l}.bin", h + "mlp.c_fc.weight", (D, F)), (f"fc1_b_{l}.bin", h + "mlp.c_fc.bias", (F,)),
            (f"fc2_w_{l}.bin", h + "mlp.c_proj.weight", (F, D)), (f"fc2_b_{l}.bin", h + "mlp.c_proj.bias", (D,)),
        ]
    files += [("ln_f_w.bin", "ln_f.weight", (D,)), ("ln_f_b.bin", "ln_f.bias", (D,))]
    return files


def write_reference_bins(model_dir: str, out_dir: str, require_reference_sizes: bool = True) -> Dict[str, int]:
    """Write every tensor of ``model_dir`` (config.json + safetensors) as ``out_dir/<name>.bin``.

    Returns {file name: number of floats}.  Raises ValueError when the model is not a GPT-2 the
    reference can run (other sizes, an untied head, another activation, another epsilon) unless
    ``require_reference_sizes`` is False (then only the layout is written, for tests)."""
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        cfg = json.load(f)
    D, L, V, P = int(cfg["n_embd"]), int(cfg["n_layer"]), int(cfg["vocab_size"]), int(cfg["n_positions"])
    F = int(cfg.get("n_inner") or 4 * D)
    if require_reference_sizes:
        got = dict(n_layer=L, n_embd=D, n_head=int(cfg["n_head"]), n_inner=F, vocab_size=V, n_positions=P)
        if got != REFERENCE_SIZES:
            diff = {k: (got[k], REFERENCE_SIZES[k]) for k in got if got[k] != REFERENCE_SIZES[k]}
            raise ValueError(f"the reference is compiled for GPT-2 small only; (given, needed): {diff}")
        if cfg.get("activation_function", "gelu_new") not in ("gelu_new", "gelu_pytorch_tanh"):
            raise ValueError("the reference computes the tanh form of GELU only (src/kernels/gemm.cu:17-20)")
        if cfg.get("scale_attn_by_inverse_layer_idx", False) or not cfg.get("tie_word_embeddings", True):
            raise ValueError("the reference has a tied head and no per-layer attention scale")
        if abs(float(cfg.get("layer_norm_epsilon", 1e-5)) - 1e-5) > 1e-12:
            raise ValueError("the reference's LayerNorm epsilon is 1e-5 (include/kernels/layernorm.cuh:23)")
    os.makedirs(out_dir, exist_ok=True)
    written: Dict[str, int] = {}
    with Checkpoint(model_dir) as ck:
        for fname, tname, shape in reference_bin_files(L, D, F, V, P):
            name = tname if tname in ck else "transformer." + tname
            if name not in ck:
                raise ValueError(f"{ck.path}: tensor {tname!r} is missing")
            t = ck.tensor(name)
            if tuple(t.shape) != shape:
                raise ValueError(f"{tname}: shape {tuple(t.shape)}, the reference reads {shape}")
            a = t.to(torch.float32).contiguous().numpy().astype("<f4", copy=False)
            a.tofile(os.path.join(out_dir, fname))
            written[fname] = int(a.size)
    return written
