"""Shared pieces of the tests: the two tiny configurations, model folders with
weights made so that faults show, the replay harness, the comparison rule."""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")

# Two tiny GPT-2 configurations that differ in every size and option.
CONFIG_A = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=64, n_head=4,
                n_inner=256, vocab_size=512, n_positions=128, layer_norm_epsilon=1e-5,
                activation_function="gelu_new", scale_attn_by_inverse_layer_idx=False, eos_token_id=511)
CONFIG_B = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=3, n_embd=96, n_head=3,
                n_inner=320, vocab_size=1000, n_positions=256, layer_norm_epsilon=1e-6,
                activation_function="gelu", scale_attn_by_inverse_layer_idx=True, eos_token_id=999)
# A third one with heads of 64 and room for long prompts: the sizes at which the tensor-memory attention
# kernel (128-query tiles, 128-key blocks) takes over from the others.
CONFIG_C = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=128, n_head=2,
                n_inner=192, vocab_size=300, n_positions=704, layer_norm_epsilon=1e-5,
                activation_function="gelu_new", scale_attn_by_inverse_layer_idx=True, eos_token_id=299)
PAGE_SIZE = {"A": 16, "B": 8, "C": 32}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}


def make_tensors(cfg: dict, seed: int, sharp: bool = True) -> Dict[str, torch.Tensor]:
    """GPT-2 tensors by checkpoint name, float32.

    ``sharp``: the attention projections are scaled up so that the softmax is far
    from uniform (single far keys carry weight, so a wrong page, a wrong mask edge or
    a stale slot changes the logits visibly), norms get random gains and every
    bias is non-zero.
    """
    g = torch.Generator().manual_seed(seed)
    D, L, F, V, P = cfg["n_embd"], cfg["n_layer"], cfg["n_inner"] or 4 * cfg["n_embd"], cfg["vocab_size"], cfg["n_positions"]

    def normal(*shape, std):
        return torch.empty(*shape).normal_(0.0, std, generator=g)

    t: Dict[str, torch.Tensor] = {}
    t["wte.weight"] = normal(V, D, std=0.5 if sharp else 0.02)
    t["wpe.weight"] = normal(P, D, std=0.5 if sharp else 0.02)
    for l in range(L):
        p = f"h.{l}."
        t[p + "ln_1.weight"] = 1.0 + normal(D, std=0.2 if sharp else 0.0)
        t[p + "ln_1.bias"] = normal(D, std=0.1 if sharp else 0.0)
        t[p + "attn.c_attn.weight"] = normal(D, 3 * D, std=(2.0 / math.sqrt(D)) if sharp else 0.02)
        t[p + "attn.c_attn.bias"] = normal(3 * D, std=0.1 if sharp else 0.0)
        t[p + "attn.c_proj.weight"] = normal(D, D, std=(0.7 / math.sqrt(D)) if sharp else 0.02)
        t[p + "attn.c_proj.bias"] = normal(D, std=0.1 if sharp else 0.0)
        t[p + "ln_2.weight"] = 1.0 + normal(D, std=0.2 if sharp else 0.0)
        t[p + "ln_2.bias"] = normal(D, std=0.1 if sharp else 0.0)
        t[p + "mlp.c_fc.weight"] = normal(D, F, std=(1.0 / math.sqrt(D)) if sharp else 0.02)
        t[p + "mlp.c_fc.bias"] = normal(F, std=0.1 if sharp else 0.0)
        t[p + "mlp.c_proj.weight"] = normal(F, D, std=(0.7 / math.sqrt(F)) if sharp else 0.02)
        t[p + "mlp.c_proj.bias"] = normal(D, std=0.1 if sharp else 0.0)
    t["ln_f.weight"] = 1.0 + normal(D, std=0.2 if sharp else 0.0)
    t["ln_f.bias"] = normal(D, std=0.1 if sharp else 0.0)
    return t


def write_model(folder: str, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> str:
    """A model folder written with the safetensors library (not the package's writer)."""
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
    return folder


def make_model(folder: str, which: str, seed: int = 0, dtype=torch.float32, sharp: bool = True) -> str:
    cfg = CONFIGS[which]
    return write_model(folder, cfg, make_tensors(cfg, seed, sharp), dtype)


def random_ids(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class Replay:
    """Drives bin/trace_run as a child process, one step at a time."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: Optional[int] = None,
                 extra: Sequence[str] = (), graphs: Optional[str] = None):
        self.out_dir = out_dir
        self.stats_path = os.path.join(out_dir, "stats.json")
        cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
               "--max-tokens", str(max_tokens), "--stats", self.stats_path]
        if page_size is not None:
            cmd += ["--page-size", str(page_size)]
        if graphs is not None:                      # "on" (the default, as generation runs), "off", "every-step"
            cmd += ["--cuda-graphs", graphs]
        cmd += list(extra)
        self.p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.n = 0
        with open(os.path.join(model_dir, "config.json")) as f:
            self.vocab = json.load(f)["vocab_size"]

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want).  Returns [wanted, vocab] float32 or None."""
        rec = {"step": self.n, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.p.stdin.write(json.dumps(rec) + "\n")
        self.p.stdin.flush()
        line = self.p.stdout.readline().strip()
        if line != f"done {self.n}":
            rest = self.p.stdout.read()
            raise RuntimeError(f"trace_run answered {line!r} {rest!r} (exit {self.p.poll()})")
        wanted = sum(len(w) for _, _, w in entries)
        out = None
        if wanted:
            out = np.fromfile(os.path.join(self.out_dir, f"{self.n}.f32"), dtype="<f4").reshape(wanted, self.vocab)
        self.n += 1
        return out

    def close(self) -> int:
        self.p.stdin.close()
        rc = self.p.wait(timeout=120)
        self.stats = {}
        if rc == 0 and os.path.isfile(self.stats_path):
            with open(self.stats_path) as f:
                self.stats = json.load(f)
        return rc


# The comparison rule of the model-level tests.  Fixed; never widened to pass.
#   float32 : weights and arithmetic are 32-bit against a float64 oracle.
#   bfloat16: both sides use the same bfloat16 weights and both keep the activations
#             handed from kernel to kernel in bfloat16 (plain_gpt2's ``store``); what
#             is left is the engine's 32-bit arithmetic against float64, and values
#             that fall on the other side of a bfloat16 rounding edge.  One such flip
#             moves a stored value by 2^-8 of itself and, with the sharp test weights,
#             a row of logits by up to 4e-3: the plain implementation run in float32
#             differs from itself in float64 by 3.6e-3 at worst on these models
#             (median 5e-8).  The limit allows two to three such flips.
TOL = {"float32": dict(fro=2e-5, peak=1e-4), "bfloat16": dict(fro=1e-2, peak=2e-2)}


def oracle_store(dtype: str):
    import plain_gpt2
    return plain_gpt2.to_bf16 if dtype == "bfloat16" else plain_gpt2._keep


def assert_close(got, want, dtype: str, what: str = ""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    tol = TOL[dtype]
    scale = max(np.abs(want).max(), 1e-6)
    for r in range(got.shape[0]):
        fro = np.linalg.norm(got[r] - want[r]) / max(np.linalg.norm(want[r]), 1e-12)
        peak = np.abs(got[r] - want[r]).max() / scale
        assert fro <= tol["fro"] and peak <= tol["peak"], (
            f"{what}: row {r}: relative error {fro:.3e} (limit {tol['fro']:.0e}), "
            f"peak {peak:.3e} (limit {tol['peak']:.0e})")
