"""The plain implementation checked against itself and against the reference's
own NumPy statements of single kernels (no GPU)."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_gpt2
from helpers import CONFIG_A, CONFIG_B, make_tensors, random_ids, write_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_causality_and_prefix_property(tmp_path):
    d = write_model(str(tmp_path / "m"), CONFIG_B, make_tensors(CONFIG_B, 2))
    cfg, w = plain_gpt2.read_model(d)
    ids = random_ids(40, cfg["vocab_size"], 1)
    full = plain_gpt2.forward_logits(cfg, w, ids)
    part = plain_gpt2.forward_logits(cfg, w, ids[:17])
    assert torch.allclose(full[:17], part, atol=1e-10)
    ids2 = list(ids)
    ids2[30] = (ids2[30] + 1) % cfg["vocab_size"]
    other = plain_gpt2.forward_logits(cfg, w, ids2)
    assert torch.allclose(full[:30], other[:30], atol=1e-10) and not torch.allclose(full[30:], other[30:], atol=1e-3)


def test_parts_against_independent_formulas():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 24, generator=g, dtype=torch.float64)
    gamma, beta = torch.randn(24, generator=g, dtype=torch.float64), torch.randn(24, generator=g, dtype=torch.float64)
    want = torch.nn.functional.layer_norm(x, (24,), gamma, beta, 1e-6)
    assert torch.allclose(plain_gpt2.layer_norm(x, gamma, beta, 1e-6), want, atol=1e-12)
    v = torch.linspace(-6, 6, 101, dtype=torch.float64)
    assert torch.allclose(plain_gpt2.gelu_erf(v), torch.nn.functional.gelu(v), atol=1e-12)
    assert torch.allclose(plain_gpt2.gelu_tanh(v), torch.nn.functional.gelu(v, approximate="tanh"), atol=1e-9)
    # attention: one head by hand
    qkv = torch.randn(6, 3 * 8, generator=g, dtype=torch.float64)
    out = plain_gpt2.causal_attention(qkv, n_head=2, scale=0.5)
    q, k, vv = qkv[:, 4:8], qkv[:, 12:16], qkv[:, 20:24]          # head 1
    for i in range(6):
        s = (k[:i + 1] @ q[i]) * 0.5
        p = torch.softmax(s, 0)
        assert torch.allclose(out[i, 4:8], p @ vv[:i + 1], atol=1e-12)
    # window of 3: only the last three keys
    outw = plain_gpt2.causal_attention(qkv, n_head=2, scale=0.5, window=3)
    i = 5
    s = (k[3:6] @ q[i]) * 0.5
    assert torch.allclose(outw[i, 4:8], torch.softmax(s, 0) @ vv[3:6], atol=1e-12)


def test_sampling_rules():
    row = torch.tensor([0.1, 3.0, 3.0, -1.0])
    assert plain_gpt2.greedy_token(row) == 1                        # lowest id among equals
    p = torch.softmax(row.double() / 0.7, 0)
    c = torch.cumsum(p, 0)
    for u in (0.0, 0.2, 0.49, 0.51, 0.999999):
        want = int((c > u).nonzero()[0, 0])
        assert plain_gpt2.temperature_token(row, 0.7, u) == want


def test_against_the_reference_numpy_oracles():
    """tests/golden/reference_kernels.npz holds outputs of the reference's own NumPy kernel
    oracles (tests/kernels/*/gen.py), made by tests/golden/make_golden.py."""
    g = np.load(os.path.join(GOLDEN, "reference_kernels.npz"))
    t64 = lambda a: torch.tensor(np.asarray(a), dtype=torch.float64)
    got = plain_gpt2.layer_norm(t64(g["layernorm_x"]), t64(g["layernorm_gamma"]), t64(g["layernorm_beta"]),
                                float(g["layernorm_eps"]))
    assert np.abs(got.numpy() - g["layernorm_y"]).max() < 1e-5          # tests/cpp/test_layernorm.cu allows 1e-4
    got = plain_gpt2.gelu_tanh(t64(g["gelu_x"]))
    assert np.abs(got.numpy() - g["gelu_y"]).max() < 1e-5
    V, P, D = (int(v) for v in g["embedding_dims"])
    wte = np.array([[t * 0.01 + d * 0.0001 for d in range(D)] for t in range(V)], dtype=np.float32)
    wpe = np.array([[p * 0.001 + d * 0.00001 for d in range(D)] for p in range(P)], dtype=np.float32)
    got = plain_gpt2.embed(g["embedding_tokens"].tolist(), t64(wte), t64(wpe))
    assert np.abs(got.numpy() - g["embedding_y"]).max() < 1e-6
    M, K, N = (int(v) for v in g["linear_dims"])
    rng = np.random.default_rng(0)                                      # tests/kernels/linear/gen.py draws these
    x = rng.normal(0, 0.02, size=(M, K)).astype(np.float32)
    w = rng.normal(0, 0.02, size=(K, N)).astype(np.float32)
    b = rng.normal(0, 0.02, size=(N,)).astype(np.float32)
    got = plain_gpt2.conv1d(t64(x), t64(w), t64(b))
    assert np.abs(got.numpy() - g["linear_y"]).max() < 1e-6
