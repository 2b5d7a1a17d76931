"""Plain, slow GPT-2 forward pass used as the oracle of the tests.

It rests on the formulas of taejuk/mini-llm's CUDA sources (cited per function
by file:line); the reference's model code is CUDA-only with its sizes fixed at
compile time (include/constants.h:5-10), so it cannot be built at the tiny test
sizes or imported on a CPU, and nothing here was compared with a run of it.
The reference's own NumPy restatements of single kernels
(tests/kernels/*/gen.py) do run on a CPU; tests/golden/ holds a comparison of
the functions below with those formulas.

Whole sequences, no cache, one function per part, float64 by default.  It
shares no code with the package: it reads model.safetensors through the
``safetensors`` library and the config.json keys directly.

``store``: an engine that serves in bfloat16 keeps the activations it hands
from one kernel to the next in bfloat16 (the normed rows, Q/K/V, the attention
output, the MLP's hidden row); the residual stream, the softmax and all sums stay
wider.  Passing ``store=to_bf16`` rounds exactly those stored values here, so that
the comparison measures the engine's arithmetic and not the storage format.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_model(model_dir: str, dtype=torch.float64):
    """config.json as a dict and every tensor of model.safetensors as ``dtype``."""
    from safetensors import safe_open

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for k in f.keys():
            name = k[len("transformer."):] if k.startswith("transformer.") else k
            tensors[name] = f.get_tensor(k).to(dtype)
    return cfg, tensors


def embed(ids: Sequence[int], wte: torch.Tensor, wpe: torch.Tensor, start: int = 0) -> torch.Tensor:
    """x[t] = wte[id_t] + wpe[pos_t] (src/kernels/embedding.cu:23-43;
    positions count from 0 inside each request, src/model/gpt2_model.cu:379-386)."""
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    pos = torch.arange(start, start + len(ids), dtype=torch.long)
    return wte[ids_t] + wpe[pos]


def layer_norm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float) -> torch.Tensor:
    """mean; biased variance of the centred values; (x-mean)*rsqrt(var+eps)*gamma+beta
    (src/kernels/layernorm.cu:32-49)."""
    mean = x.sum(dim=-1, keepdim=True) / x.shape[-1]
    centred = x - mean
    var = (centred * centred).sum(dim=-1, keepdim=True) / x.shape[-1]
    return centred / torch.sqrt(var + eps) * gamma + beta


def conv1d(x: torch.Tensor, w_in_out: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """y = x @ W + b with W stored [in, out] as GPT-2's Conv1D keeps it
    (scripts/export_weights.py:48-52; src/kernels/linear.cu:8-26)."""
    return x @ w_in_out + b


def gelu_tanh(v: torch.Tensor) -> torch.Tensor:
    """0.5*v*(1+tanh(0.7978845608*(v+0.044715*v^3))) (src/kernels/gemm.cu:17-20)."""
    return 0.5 * v * (1.0 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)))


def gelu_erf(v: torch.Tensor) -> torch.Tensor:
    """0.5*v*(1+erf(v/sqrt(2))): the "gelu" value of activation_function; the
    reference has only the tanh form (src/kernels/gelu.cu:7-30)."""
    return 0.5 * v * (1.0 + torch.erf(v / math.sqrt(2.0)))


def activation(name: str):
    if name in ("gelu_new", "gelu_pytorch_tanh", "gelu_fast"):
        return gelu_tanh
    if name == "gelu":
        return gelu_erf
    raise ValueError(f"activation {name!r}")


def causal_attention(qkv: torch.Tensor, n_head: int, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """Multi-head causal attention of one whole sequence.

    qkv columns are Q | K | V thirds, head h = columns h*dh..h*dh+dh-1 of each
    third (src/kernels/prefill/flashattention.cu:60-64,100-111); score =
    (q.k)*scale, keys k <= query only, softmax over them, weighted sum of V
    (src/kernels/prefill/flashattention.cu:129-168 as an online softmax;
    src/kernels/decode/paged_attention.cu:60-120 as a two-pass softmax, whose
    +1e-6 on the denominator is left out here).
    ``window``: if given, a query at i sees keys i-window+1..i only.
    """
    T, three_d = qkv.shape
    D = three_d // 3
    dh = D // n_head
    q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
    out = torch.empty(T, D, dtype=qkv.dtype)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= idx[None, :] > (idx[:, None] - window)
    for h in range(n_head):
        sl = slice(h * dh, (h + 1) * dh)
        s = (q[:, sl] @ k[:, sl].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, sl] = p @ v[:, sl]
    return out


def to_bf16(t: torch.Tensor) -> torch.Tensor:
    """Round to the nearest bfloat16 value, keep the dtype."""
    return t.to(torch.bfloat16).to(t.dtype)


def _keep(t: torch.Tensor) -> torch.Tensor:
    return t


def block(x: torch.Tensor, w: Dict[str, torch.Tensor], l: int, cfg: dict, store=_keep) -> torch.Tensor:
    """One pre-LayerNorm block: x += proj(attn(ln_1(x))); x += mlp(ln_2(x))
    (src/model/gpt2_model.cu:271-365)."""
    eps = float(cfg.get("layer_norm_epsilon", 1e-5))
    n_head = int(cfg["n_head"])
    D = int(cfg["n_embd"])
    dh = D // n_head
    scale = 1.0 / math.sqrt(dh) if cfg.get("scale_attn_weights", True) else 1.0
    if cfg.get("scale_attn_by_inverse_layer_idx", False):
        scale = scale / float(l + 1)
    p = f"h.{l}."
    h = store(layer_norm(x, w[p + "ln_1.weight"], w[p + "ln_1.bias"], eps))
    qkv = store(conv1d(h, w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]))
    a = store(causal_attention(qkv, n_head, scale))
    x = x + conv1d(a, w[p + "attn.c_proj.weight"], w[p + "attn.c_proj.bias"])
    h = store(layer_norm(x, w[p + "ln_2.weight"], w[p + "ln_2.bias"], eps))
    act = activation(cfg.get("activation_function", "gelu_new"))
    f = store(act(conv1d(h, w[p + "mlp.c_fc.weight"], w[p + "mlp.c_fc.bias"])))
    x = x + conv1d(f, w[p + "mlp.c_proj.weight"], w[p + "mlp.c_proj.bias"])
    return x


def lm_head(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict, store=_keep) -> torch.Tensor:
    """logits = ln_f(x) @ wte^T, no bias (src/model/gpt2_model.cu:410-428);
    an untied model multiplies by lm_head.weight instead."""
    eps = float(cfg.get("layer_norm_epsilon", 1e-5))
    y = store(layer_norm(x, w["ln_f.weight"], w["ln_f.bias"], eps))
    if cfg.get("tie_word_embeddings", True) or "lm_head.weight" not in w:
        return y @ w["wte.weight"].T
    return y @ w["lm_head.weight"].T


def forward_logits(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], store=_keep) -> torch.Tensor:
    """Logits at every position of one whole sequence, [len(ids), vocab]."""
    x = embed(ids, w["wte.weight"], w["wpe.weight"])
    for l in range(int(cfg["n_layer"])):
        x = block(x, w, l, cfg, store)
    return lm_head(x, w, cfg, store)


def logits_at(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], rows: Sequence[int], store=_keep) -> torch.Tensor:
    """Logits at the chosen positions of one whole sequence, [len(rows), vocab]: the blocks run over the
    whole sequence, the final norm and the head only on the chosen rows, as the reference does it for
    the last row of a prompt (src/model/gpt2_model.cu:408-428).  For wide vocabularies."""
    x = embed(ids, w["wte.weight"], w["wpe.weight"])
    for l in range(int(cfg["n_layer"])):
        x = block(x, w, l, cfg, store)
    return lm_head(x[torch.as_tensor(list(rows), dtype=torch.long)], w, cfg, store)


def hidden_states(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> List[torch.Tensor]:
    """The residual stream after the embedding and after every block."""
    x = embed(ids, w["wte.weight"], w["wpe.weight"])
    out = [x]
    for l in range(int(cfg["n_layer"])):
        x = block(x, w, l, cfg)
        out.append(x)
    return out


def greedy_token(logits_row: torch.Tensor) -> int:
    """argmax, the lowest id among equals (src/kernels/argmax.cu:12-20)."""
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def temperature_token(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """Inverse-CDF draw from softmax(logits/temperature) with the uniform u in [0,1):
    the first id whose cumulative probability exceeds u.  (The reference samples
    by argmax only, README.md "Current Limitations".)"""
    z = logits_row.to(torch.float64) / temperature
    p = torch.exp(z - z.max())
    c = torch.cumsum(p, dim=0)
    target = u * float(c[-1])
    idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64), right=True))
    return min(idx, logits_row.numel() - 1)


def generate_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int,
                    stop_at_eos: bool = False, store=_keep) -> List[int]:
    """Greedy continuation by whole-sequence recomputation (no cache)."""
    ids = list(prompt)
    out: List[int] = []
    eos = cfg.get("eos_token_id", None)
    for _ in range(n_new):
        if len(ids) >= int(cfg["n_positions"]):
            break
        tok = greedy_token(forward_logits(cfg, w, ids, store)[-1])
        out.append(tok)
        ids.append(tok)
        if stop_at_eos and eos is not None and tok == eos:
            break
    return out
