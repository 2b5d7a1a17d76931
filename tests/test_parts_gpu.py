"""Each part of the model alone, built from its constants, against the plain functions."""
import math

import pytest
import torch

import plain_gpt2

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


class Rt:
    def __init__(self, dtype):
        from mini_llm_b200 import ops
        self.dtype, self.device, self.ops = dtype, DEV, ops

    @property
    def act_dtype(self):
        return self.dtype


class Ctx:
    def __init__(self, T):
        from mini_llm_b200.engine.context import Workspace
        self.ws = Workspace(DEV, 256)
        self.T = T


def close(got, want, dtype, f32=2e-5, bf16_ulps=1.0):
    """float32: absolute/relative 2e-5-like bound; bfloat16: within `bf16_ulps` units in the last
    place of the result's magnitude (one unit = 2^-8 of the value) plus the same small floor."""
    got, want = got.double().cpu(), want.double().cpu()
    mag = want.abs().clamp(min=1.0)
    if dtype == torch.float32:
        return bool(((got - want).abs() / mag).max() < f32)
    return bool(((got - want).abs() / mag).max() < bf16_ulps * 2 ** -8)


def rnd(*shape, seed, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,eps", [(80, 1e-5), (1600, 1e-6)])
def test_layernorm_part(dtype, D, eps):
    from mini_llm_b200.parts.norm import LayerNorm
    part = LayerNorm(hidden_size=D, eps=eps)
    g, b, x = rnd(D, seed=1) + 1, rnd(D, seed=2), rnd(33, D, seed=3, scale=2.0) + 0.7
    part.bind({"weight": g.to(DEV), "bias": b.to(DEV)}, Rt(dtype))
    got = part.forward(x.to(DEV), Ctx(33))
    want = plain_gpt2.layer_norm(x.double(), g.double(), b.double(), eps)
    assert got.dtype == dtype
    assert close(got, want, dtype)
    rows = torch.tensor([32, 0, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(part.forward(x.to(DEV), Ctx(33), rows=rows).cpu(), got.cpu()[[32, 0, 5]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act,fn", [("gelu_tanh", plain_gpt2.gelu_tanh), ("gelu_erf", plain_gpt2.gelu_erf)])
@pytest.mark.parametrize("T", [5, 130])
def test_mlp_part(dtype, act, fn, T):
    from mini_llm_b200.parts.mlp import MLP
    D, F = 96, 320
    part = MLP(hidden_size=D, inner_size=F, activation=act)
    w1, b1, w2, b2 = rnd(F, D, seed=1, scale=D ** -0.5), rnd(F, seed=2), rnd(D, F, seed=3, scale=F ** -0.5), rnd(D, seed=4)
    part.bind({"fc_weight": w1.to(dtype).to(DEV), "fc_bias": b1.to(DEV), "proj_weight": w2.to(dtype).to(DEV),
               "proj_bias": b2.to(DEV)}, Rt(dtype))
    h = rnd(T, D, seed=5).to(dtype)
    x = rnd(T, D, seed=6).to(DEV)
    x0 = x.clone()
    part.forward(h.to(DEV), Ctx(T), x)
    store = plain_gpt2.to_bf16 if dtype == torch.bfloat16 else plain_gpt2._keep
    W1, W2 = w1.to(dtype).double(), w2.to(dtype).double()
    mid = store(fn(h.double() @ W1.t() + b1.double()))
    want = x0.double().cpu() + mid @ W2.t() + b2.double()
    assert close(x, want, dtype, f32=3e-5, bf16_ulps=2.0)       # two products in a row
    with pytest.raises(ValueError):
        MLP(hidden_size=8, inner_size=8, activation="relu")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_positions_and_head_parts(dtype):
    from mini_llm_b200.parts.embedding import TokenEmbedding
    from mini_llm_b200.parts.head import TiedHead
    from mini_llm_b200.parts.positions import LearnedPositions, NoPositions
    V, P, D, T = 101, 40, 48, 9
    wte, wpe = rnd(V, D, seed=1), rnd(P, D, seed=2)
    emb, pos, head = TokenEmbedding(hidden_size=D, vocab_size=V), LearnedPositions(hidden_size=D, max_positions=P), TiedHead(D, V)
    rt = Rt(dtype)
    emb.bind({"table": wte.to(dtype).to(DEV)}, rt)
    pos.bind({"table": wpe.to(dtype).to(DEV)}, rt)
    head.bind({}, rt)
    head.tie(emb)
    ctx = Ctx(T)
    ids = [5, 100, 0, 7, 7, 33, 2, 1, 99]
    ctx.token_ids = torch.tensor(ids, dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor([3, 4, 5, 0, 1, 2, 39, 0, 17], dtype=torch.int32, device=DEV)
    x = emb.forward(ctx, pos)
    want = wte.to(dtype).double()[ids] + wpe.to(dtype).double()[ctx.positions.cpu().long()]
    assert x.dtype == torch.float32 and (x.double().cpu() - want).abs().max() < 1e-6
    x2 = emb.forward(ctx, NoPositions())
    assert (x2.double().cpu() - wte.to(dtype).double()[ids]).abs().max() < 1e-6
    assert pos.max_positions == P and NoPositions().max_positions is None
    y = rnd(4, D, seed=3).to(dtype).to(DEV)
    logits = head.forward(y, ctx)
    assert logits.dtype == torch.float32 and tuple(logits.shape) == (4, V)
    assert close(logits, y.double().cpu() @ wte.to(dtype).double().t(), dtype, bf16_ulps=0.5)   # 32-bit logits


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,window", [(4, 4, 16, None), (3, 3, 32, None), (4, 2, 32, None), (2, 2, 64, 10)])
def test_attention_part_over_its_cache(dtype, H, Hkv, dh, window):
    """The attention part alone: a 50-token request fed in portions of 20, 1, 1, 28 through its
    own pages, against plain causal attention (also with fewer key/value heads and a window)."""
    from mini_llm_b200.cache.manager import CacheManager
    from mini_llm_b200.engine.context import StepContext, StepLayout, Workspace, attention_tiles, pack_step
    from mini_llm_b200.parts.attention import Attention
    from mini_llm_b200.parts.model import LayerCache
    import numpy as np
    D, T, page = 64, 50, 8
    scale = 0.3
    part = Attention(hidden_size=D, num_heads=H, head_dim=dh, scale=scale, num_kv_heads=Hkv, window=window)
    qs, kvs = H * dh, Hkv * dh
    wq, bq = rnd(qs + 2 * kvs, D, seed=1, scale=2 * D ** -0.5), rnd(qs + 2 * kvs, seed=2, scale=0.1)
    wo, bo = rnd(D, qs, seed=3, scale=qs ** -0.5), rnd(D, seed=4, scale=0.1)
    part.bind({"qkv_weight": wq.to(dtype).to(DEV), "qkv_bias": bq.to(DEV), "out_weight": wo.to(dtype).to(DEV),
               "out_bias": bo.to(DEV)}, Rt(dtype))
    cm = CacheManager({0: part.cache_need()}, page_size=page, num_pages=16, max_num_seqs=2, dtype=dtype, device=DEV)
    cm.admit("r")
    h = rnd(T, D, seed=5).to(dtype)
    ws = Workspace(DEV, 64)
    out = torch.zeros(T, D, device=DEV)
    pos = 0
    for n in (20, 1, 1, 28):
        assert cm.reserve("r", n)
        tiles = [] if n == 1 else attention_tiles([n])
        lay = StepLayout.make(n, 1, 0, [16], len(tiles) // 3)
        host = np.zeros(lay.total, dtype=np.int32)
        pack_step(lay, host, token_ids=[0] * n, positions=list(range(pos, pos + n)), token_seq=[0] * n, logit_rows=[],
                  state_slots=[0], cu_q=[0, n], q_start=[pos], ctx_len=[pos + n],
                  slot_mappings=[cm.slots_for("r", 0, pos, n)], block_tables=[[cm.table("r", 0)]], attn_tiles=tiles)
        ctx = StepContext(lay, torch.from_numpy(host).to(DEV), ws, q_lens=[n], q_starts=[pos])
        g = cm.groups[0]
        cache = LayerCache(group=0, k_pages=g.pool[0, 0], v_pages=g.pool[0, 1])
        part.forward(h[pos:pos + n].to(DEV), ctx, cache, out[pos:pos + n])
        cm.commit("r", n)
        pos += n
    # plain: project, attend causally (grouped heads, optional window), project back
    store = plain_gpt2.to_bf16 if dtype == torch.bfloat16 else plain_gpt2._keep
    qkv = store(h.double() @ wq.to(dtype).double().t() + bq.double())
    q, k, v = qkv[:, :qs], qkv[:, qs:qs + kvs], qkv[:, qs + kvs:]
    att = torch.zeros(T, qs, dtype=torch.float64)
    idx = torch.arange(T)
    vis = idx[None, :] <= idx[:, None]
    if window:
        vis &= idx[None, :] > idx[:, None] - window
    for hh in range(H):
        hk = hh // (H // Hkv)
        s = (q[:, hh * dh:(hh + 1) * dh] @ k[:, hk * dh:(hk + 1) * dh].t()) * scale
        att[:, hh * dh:(hh + 1) * dh] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, hk * dh:(hk + 1) * dh]
    want = store(att) @ wo.to(dtype).double().t() + bo.double()
    assert close(out, want, dtype, f32=5e-5, bf16_ulps=4.0)   # bfloat16: Q/K/V and the attention output are stored rounded
    if window:
        assert cm.groups[0].allocator.num_in_use < (T + page - 1) // page       # pages behind the window went back
