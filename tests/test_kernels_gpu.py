"""Each kernel alone against a plain PyTorch float32/float64 statement of the same
operation, at sizes other than the engine's test models."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mini_llm_b200 import ops as o
    o.library()
    return o


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,D,V,P", [(7, 48, 33, 20), (130, 1600, 101, 140), (1, 80, 5, 3)])
def test_embed(ops, dtype, T, D, V, P):
    table, pos_table = rnd(V, D, seed=1, dtype=dtype), rnd(P, D, seed=2, dtype=dtype)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    pos = torch.randint(0, P, (T,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(T, D, device=DEV)
    ops.embed(ids, pos, table, pos_table, out)
    want = table.float()[ids.long()] + pos_table.float()[pos.long()]
    assert torch.equal(out, want)
    ops.embed(ids, pos, table, None, out)
    assert torch.equal(out, table.float()[ids.long()])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,D,eps", [(5, 48, 1e-5), (33, 1600, 1e-6), (3, 1000, 1e-3), (2, 4096, 1e-5)])
def test_layernorm(ops, out_dtype, R, D, eps):
    x = rnd(R, D, seed=4, scale=3.0) + 1.5
    gamma, beta = rnd(D, seed=5) + 1.0, rnd(D, seed=6)
    out = torch.empty(R, D, device=DEV, dtype=out_dtype)
    ops.layernorm(x, gamma, beta, eps, out)
    want = torch.nn.functional.layer_norm(x.double(), (D,), gamma.double(), beta.double(), eps)
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    assert (out.double() - want).abs().max() < tol * max(1.0, want.abs().max().item())
    # gathered rows
    rows = torch.tensor([R - 1, 0, R - 1], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, D, device=DEV, dtype=out_dtype)
    ops.layernorm(x, gamma, beta, eps, out2, rows=rows)
    assert torch.equal(out2, out[rows.long()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 50, 33), (67, 79, 37), (130, 200, 96), (5, 1003, 768), (64, 64, 16),
                                   (300, 260, 72), (2048, 768, 96), (257, 1003, 40)])
def test_linear_and_epilogues(ops, dtype, M, N, K):
    x, w, b = rnd(M, K, seed=7, dtype=dtype), rnd(N, K, seed=8, scale=K ** -0.5, dtype=dtype), rnd(N, seed=9)
    ref = x.double() @ w.double().t()
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    out = torch.empty(M, N, device=DEV, dtype=dtype)
    ops.linear(x, w, None, out=out)
    assert (out.double() - ref).abs().max() < tol * 4
    ops.linear(x, w, b, out=out, act="gelu_tanh")
    want = torch.nn.functional.gelu(ref + b.double(), approximate="tanh")
    assert (out.double() - want).abs().max() < tol * 4
    ops.linear(x, w, b, out=out, act="gelu_erf")
    want = torch.nn.functional.gelu(ref + b.double())
    assert (out.double() - want).abs().max() < tol * 4
    acc = rnd(M, N, seed=10)
    acc0 = acc.clone()
    ops.linear(x, w, b, out=acc, accumulate=True)                   # 32-bit residual stream
    assert (acc.double() - (acc0.double() + ref + b.double())).abs().max() < 2e-5 * 8
    # a column slice as input and a padded output
    wide = rnd(M, K + 24, seed=11, dtype=dtype)
    xs = wide[:, 8:8 + K]
    big = torch.zeros(M, N + 5, device=DEV, dtype=torch.float32)
    ops.linear(xs, w, None, out=big[:, :N])
    assert (big[:, :N].double() - xs.double() @ w.double().t()).abs().max() < 2e-5 * 8
    assert torch.all(big[:, N:] == 0)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 768, 768), (8, 2304, 768), (3, 50, 40), (17, 1003, 96), (64, 320, 3072),
                                   (33, 50257, 64), (64, 9472 + 5, 128), (5, 16, 8)])
def test_linear_small_m_against_the_plain_kernel(ops, out_dtype, M, N, K):
    """The weight-streaming tensor-core product beside its plain twin and float64."""
    dt = torch.bfloat16
    x, w, b = rnd(M, K, seed=1, dtype=dt), rnd(N, K, seed=2, scale=K ** -0.5, dtype=dt), rnd(N, seed=3)
    ref = x.double() @ w.double().t() + b.double()
    for act in (None, "gelu_tanh", "gelu_erf"):
        out = torch.full((M, N), 7.0, device=DEV, dtype=out_dtype)
        ops.linear(x, w, b, out=out, act=act, impl="smallm")
        plain = torch.empty(M, N, device=DEV, dtype=out_dtype)
        ops.linear(x, w, b, out=plain, act=act, impl="simt")
        want = ref if act is None else torch.nn.functional.gelu(ref, approximate="tanh" if act == "gelu_tanh" else "none")
        tol = 2e-5 if out_dtype == torch.float32 else 1e-2
        assert (out.double() - want).abs().max() < tol * max(1.0, want.abs().max().item())
        assert (out.double() - plain.double()).abs().max() < tol * max(1.0, want.abs().max().item())
    acc = rnd(M, N, seed=4)
    acc0 = acc.clone()
    wide = rnd(M, K + 16, seed=5, dtype=dt)
    ops.linear(wide[:, 8:8 + K], w, None, out=acc, accumulate=True, impl="smallm")
    want = acc0.double() + wide[:, 8:8 + K].double() @ w.double().t()
    assert (acc.double() - want).abs().max() < 1e-4


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(65, 64, 64), (128, 128, 64), (129, 130, 72), (300, 200, 40), (2048, 2304, 768),
                                   (2048, 768, 3072), (257, 1003, 96), (70, 50257, 128), (1000, 320, 8)])
def test_linear_tcgen05_against_the_plain_kernel(ops, out_dtype, M, N, K):
    """The TMA + tcgen05 product beside its plain twin and float64: tails in M, N and K,
    every epilogue, a sliced input, an output whose rows are not 16-byte aligned."""
    dt = torch.bfloat16
    x, w, b = rnd(M, K, seed=1, dtype=dt), rnd(N, K, seed=2, scale=K ** -0.5, dtype=dt), rnd(N, seed=3)
    ref = x.double() @ w.double().t() + b.double()
    tol = 3e-5 if out_dtype == torch.float32 else 1e-2
    for act in (None, "gelu_tanh", "gelu_erf"):
        out = torch.full((M, N), 7.0, device=DEV, dtype=out_dtype)
        ops.linear(x, w, b, out=out, act=act, impl="tcgen05")
        ops.check_device_errors()
        want = ref if act is None else torch.nn.functional.gelu(ref, approximate="tanh" if act == "gelu_tanh" else "none")
        assert (out.double() - want).abs().max() < tol * max(1.0, want.abs().max().item()), act
    plain = torch.empty(M, N, device=DEV, dtype=out_dtype)
    out = torch.empty(M, N, device=DEV, dtype=out_dtype)
    ops.linear(x, w, None, out=plain, impl="simt")
    ops.linear(x, w, None, out=out, impl="tcgen05")
    assert (out.double() - plain.double()).abs().max() < tol * max(1.0, ref.abs().max().item())
    acc = rnd(M, N, seed=4)
    acc0 = acc.clone()
    wide = rnd(M, K + 16, seed=5, dtype=dt)
    ops.linear(wide[:, 8:8 + K], w, b, out=acc, accumulate=True, impl="tcgen05")
    want = acc0.double() + wide[:, 8:8 + K].double() @ w.double().t() + b.double()
    assert (acc.double() - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item())
    pad = torch.zeros(M, N + 3, device=DEV, dtype=out_dtype)             # row stride not a multiple of 16 bytes
    ops.linear(x, w, b, out=pad[:, :N], impl="tcgen05")
    assert (pad[:, :N].double() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    assert torch.all(pad[:, N:] == 0)
    # rows 16-byte aligned but wider than N, and more rows than M: the copy engine's stores stop at the edges
    big = torch.full((M + 5, N + 8), 3.0, device=DEV, dtype=out_dtype)
    ops.linear(x, w, b, out=big[:M, :N], impl="tcgen05")
    assert (big[:M, :N].double() - ref).abs().max() < tol * max(1.0, ref.abs().max().item())
    assert torch.all(big[:, N:] == 3.0) and torch.all(big[M:] == 3.0)
    if out_dtype == torch.float32:
        big[:M, :N] = acc0
        ops.linear(wide[:, 8:8 + K], w, b, out=big[:M, :N], accumulate=True, impl="tcgen05")
        assert (big[:M, :N].double() - want).abs().max() < 1e-4 * max(1.0, want.abs().max().item())
        assert torch.all(big[:, N:] == 3.0) and torch.all(big[M:] == 3.0)
    ops.check_device_errors()


def test_linear_tcgen05_rows_do_not_depend_on_the_batch(ops):
    x, w = rnd(600, 768, seed=1, dtype=torch.bfloat16), rnd(2304, 768, seed=2, scale=0.05, dtype=torch.bfloat16)
    full = torch.empty(600, 2304, device=DEV)
    ops.linear(x, w, None, out=full, impl="tcgen05")
    for lo, hi in ((0, 65), (100, 400), (513, 600)):
        part = torch.empty(hi - lo, 2304, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="tcgen05")
        assert torch.equal(part, full[lo:hi])
    ops.check_device_errors()


@pytest.mark.parametrize("M,N,K,eps", [(1, 768, 768, 1e-5), (8, 2304, 768, 1e-5), (5, 1000, 96, 1e-6), (16, 320, 1600, 1e-5),
                                       (13, 50257, 64, 1e-3), (40, 200, 1024, 1e-5)])
def test_small_m_product_with_the_norm_fused_in(ops, M, N, K, eps):
    """LayerNorm fused into the loads of the weight-streaming product, also with gathered rows,
    against the two separate kernels."""
    from mini_llm_b200.engine.context import Workspace
    ws = Workspace(torch.device(DEV), 64)
    x = rnd(M + 3, K, seed=1, scale=2.0) + 0.5
    gamma, beta = rnd(K, seed=2) + 1.0, rnd(K, seed=3)
    w, b = rnd(N, K, seed=4, scale=K ** -0.5, dtype=torch.bfloat16), rnd(N, seed=5)
    for rows in (None, torch.tensor([(3 * i + 1) % (M + 3) for i in range(M)], dtype=torch.int32, device=DEV)):
        xin = x[:M] if rows is None else x
        normed = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
        ops.layernorm(xin, gamma, beta, eps, normed, rows=rows)
        for act, out_dtype in ((None, torch.float32), ("gelu_tanh", torch.bfloat16), ("gelu_erf", torch.bfloat16)):
            want = torch.empty(M, N, device=DEV, dtype=out_dtype)
            ops.linear(normed, w, b, out=want, act=act, impl="smallm")
            got = torch.full((M, N), 3.0, device=DEV, dtype=out_dtype)
            ops.linear(ops.NormedInput(xin, gamma, beta, eps, rows, ws, torch.bfloat16), w, b, out=got, act=act)
            # the fused norm sums a row in another order: a normed value may round to the other bfloat16 neighbour
            scale = max(1.0, want.float().abs().max().item())
            assert (got.double() - want.double()).abs().max() < (2e-3 if out_dtype == torch.float32 else 1.6e-2) * scale
        ref = torch.nn.functional.layer_norm(xin.double() if rows is None else xin.double()[rows.long()], (K,),
                                             gamma.double(), beta.double(), eps) @ w.double().t() + b.double()
        got = torch.empty(M, N, device=DEV)
        ops.linear(ops.NormedInput(xin, gamma, beta, eps, rows, ws, torch.bfloat16), w, b, out=got)
        assert (got.double() - ref).abs().max() < 2e-2 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M,H,Hkv,dh,page,K", [(1, 12, 12, 64, 16, 768), (8, 4, 4, 16, 16, 64), (13, 3, 3, 32, 8, 96),
                                               (64, 6, 2, 64, 4, 128)])
def test_small_m_qkv_product_writes_the_cache(ops, M, H, Hkv, dh, page, K):
    """The Q|K|V projection whose epilogue puts keys and values into their page slots, against
    the product followed by the copy kernel."""
    from mini_llm_b200.engine.context import Workspace
    ws = Workspace(torch.device(DEV), 64)
    q_size, kv = H * dh, Hkv * dh
    N = q_size + 2 * kv
    x = rnd(M, K, seed=1, dtype=torch.bfloat16)
    w, b = rnd(N, K, seed=2, scale=K ** -0.5, dtype=torch.bfloat16), rnd(N, seed=3)
    P = 40 + 300 // page               # room for the 300 rows of the second part
    g = torch.Generator().manual_seed(4)
    slots = torch.randperm(P * page, generator=g)[:M].to(torch.int32).to(DEV)
    qkv = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    # the reference product runs the kernel that the fused call will choose for this size
    ops.linear(x, w, b, out=qkv, impl="smallm" if ops._small_m_wins(M, N, K) else "tcgen05")
    wk = torch.full((P, Hkv, page, dh), 9.0, device=DEV, dtype=torch.bfloat16)
    wv = wk.clone()
    ops.kv_write(qkv[:, q_size:q_size + kv], qkv[:, q_size + kv:], wk, wv, slots)
    gk = torch.full((P, Hkv, page, dh), 9.0, device=DEV, dtype=torch.bfloat16)
    gv = gk.clone()
    q_buf = torch.empty(M, q_size, device=DEV, dtype=torch.bfloat16)
    q = ops.linear_qkv_cache(x, w, b, q_buf, gk, gv, slots, ws)
    assert q.data_ptr() == q_buf.data_ptr()
    assert torch.equal(q, qkv[:, :q_size]) and torch.equal(gk, wk) and torch.equal(gv, wv)
    # many rows: the tensor-memory product's epilogue (head sizes that are multiples of 32) or the product
    # followed by the copy kernel give the same cache
    M2 = 300
    x2 = rnd(M2, K, seed=5, dtype=torch.bfloat16)
    slots2 = torch.randperm(P * page, generator=g)[:M2].to(torch.int32).to(DEV)
    assert slots2.numel() == M2
    with pytest.raises(Exception):       # one slot per row, or the call is refused
        ops.linear_qkv_cache(x2, w, b, torch.empty(M2, q_size, device=DEV, dtype=torch.bfloat16), gk, gv, slots2[:-1], ws)
    gk.fill_(9.0), gv.fill_(9.0)
    q2 = ops.linear_qkv_cache(x2, w, b, torch.empty(M2, q_size, device=DEV, dtype=torch.bfloat16), gk, gv, slots2, ws)
    full = torch.empty(M2, N, device=DEV, dtype=torch.bfloat16)
    ops.linear(x2, w, b, out=full)
    assert torch.equal(q2, full[:, :q_size])
    sl = slots2.long()
    assert torch.equal(gk[sl // page, :, sl % page].reshape(M2, -1), full[:, q_size:q_size + kv])
    assert torch.equal(gv[sl // page, :, sl % page].reshape(M2, -1), full[:, q_size + kv:])
    untouched = torch.ones(P * page, dtype=torch.bool, device=DEV)
    untouched[sl] = False
    rest = gk.permute(0, 2, 1, 3).reshape(P * page, -1)[untouched]
    assert torch.all(rest == 9.0)
    ops.check_device_errors()


def test_linear_small_m_rows_do_not_depend_on_the_batch(ops):
    x, w = rnd(64, 768, seed=1, dtype=torch.bfloat16), rnd(2304, 768, seed=2, scale=0.05, dtype=torch.bfloat16)
    full = torch.empty(64, 2304, device=DEV)
    ops.linear(x, w, None, out=full, impl="smallm")
    for lo, hi in ((0, 1), (7, 9), (63, 64), (10, 40)):
        part = torch.empty(hi - lo, 2304, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="smallm")
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("M,N,K", [(1, 768, 768), (8, 2304, 768), (3, 50, 40), (16, 1003, 96), (5, 320, 3072), (13, 50257, 64),
                                   (17, 768, 3072), (40, 4800, 1600), (64, 768, 768), (64, 100, 6400), (33, 2304, 768),
                                   (9, 7, 12), (2, 1600, 6400), (64, 1024, 4096), (33, 1600, 6400), (48, 6400, 1600),
                                   (20, 50257, 1024), (64, 130, 12000), (8, 50257, 768), (16, 40000, 1600), (3, 38000, 2048),
                                   (1, 50257, 1024), (64, 50257, 768), (40, 40000, 1024), (32, 38000, 1600), (33, 38000, 1600),
                                   (8, 768, 3072), (16, 1600, 6400), (3, 1024, 4096), (64, 768, 3072), (24, 1600, 6400), (40, 1024, 4096),
                                   (5, 100, 2500), (48, 1000, 2052)])
def test_linear_stream_float32(ops, M, N, K):
    """The 32-bit weight-streaming product (weights by bulk copy into shared memory, warps own tokens, K slices
    of narrow matrices shared by a cluster; for a matrix as tall as a vocabulary and up to 16 rows the kernel that
    stays on its SM and gives each warp rows of its own) beside float64, at 1 to 64 rows."""
    x, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=K ** -0.5), rnd(N, seed=3)
    ref = x.double() @ w.double().t() + b.double()
    for act in (None, "gelu_tanh", "gelu_erf"):
        out = torch.full((M, N), 7.0, device=DEV)
        ops.linear(x, w, b, out=out, act=act, impl="stream_f32")
        want = ref if act is None else torch.nn.functional.gelu(ref, approximate="tanh" if act == "gelu_tanh" else "none")
        assert (out.double() - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    acc = rnd(M, N, seed=4)
    acc0 = acc.clone()
    wide = rnd(M, K + 8, seed=5)
    ops.linear(wide[:, 4:4 + K], w, None, out=acc, accumulate=True, impl="stream_f32")
    assert (acc.double() - (acc0.double() + wide[:, 4:4 + K].double() @ w.double().t())).abs().max() < 1e-4
    # a row does not depend on the batch: alone, in a pair, and in the whole batch it has the same bits, as long as
    # the same kernel computes it.  Which kernel that is depends on the matrix and on the side of a row count: the
    # kernel that keeps its weights in registers takes a matrix up to a count of its own (all rows that fit its shared
    # memory for a vocabulary, 16 to 48 for the layer matrices it wins at), long rows go to cluster slices where
    # those win; otherwise up to 16 rows the threads split K and beyond them the warps split the tokens.  The
    # library says which kernel takes which count; kernels differ in rounding.
    full = torch.empty(M, N, device=DEV)
    ops.linear(x, w, None, out=full, impl="stream_f32")
    kernel_of = lambda m: ops.library().mllm_linear_stream_f32_kernel_of(m, N, K)
    cuts = [(M - 1, M), (0, 1), (max(0, M - 9), M), (0, min(M, 16)), (M // 2, min(M, M // 2 + 3)), (0, min(M, 17)),
            (max(0, M - 17), M), (max(0, M - 30), M), (0, M)]
    same = [(lo, hi) for lo, hi in cuts if hi > lo and kernel_of(hi - lo) == kernel_of(M)]
    for lo, hi in same:
        part = torch.empty(hi - lo, N, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="stream_f32")
        assert torch.equal(part, full[lo:hi]), (lo, hi)
    for lo, hi in [(lo, hi) for lo, hi in cuts if hi > lo and kernel_of(hi - lo) != kernel_of(M)][:1]:
        part = torch.empty(hi - lo, N, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="stream_f32")
        assert (part.double() - full[lo:hi].double()).abs().max() < 2e-5 * max(1.0, ref.abs().max().item())
    if M <= 64:                                   # and it is what the dispatcher picks for float32 rows up to 64
        auto = torch.empty(M, N, device=DEV)
        n0 = ops.launches
        ops.linear(x, w, None, out=auto)
        assert torch.equal(auto, full) and ops.launches == n0 + 1
    ops.check_device_errors()


def test_linear_stream_float32_at_random_shapes(ops):
    """Forty shapes drawn at random (1 to 64 rows, widths and lengths that are no multiples of a tile, K in steps of 4)
    through whichever kernel the library picks for them, beside float64; bias, residual sum and GELU at every second."""
    import random
    rng = random.Random(7)
    seen = set()
    for i in range(40):
        M = rng.choice([1, 2, 3, 5, 8, 9, 15, 16, 17, 23, 24, 25, 31, 32, 33, 47, 48, 49, 63, 64])
        N = rng.choice([rng.randint(1, 300), rng.randint(300, 2400), rng.randint(2400, 7000)])
        K = 4 * rng.choice([rng.randint(1, 64), rng.randint(64, 512), rng.randint(512, 1800)])
        seen.add(ops.library().mllm_linear_stream_f32_kernel_of(M, N, K))
        x, w, b = rnd(M, K, seed=3 * i), rnd(N, K, seed=3 * i + 1, scale=K ** -0.5), rnd(N, seed=3 * i + 2)
        ref = x.double() @ w.double().t() + b.double()
        out = torch.full((M + 1, N + 1), 5.0, device=DEV)
        if i % 2:
            acc0 = rnd(M, N, seed=1000 + i)
            out[:M, :N] = acc0
            ops.linear(x, w, b, out=out[:M, :N], act="gelu_tanh", accumulate=True)
            want = acc0.double() + torch.nn.functional.gelu(ref, approximate="tanh")
        else:
            ops.linear(x, w, b, out=out[:M, :N])
            want = ref
        assert (out[:M, :N].double() - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item()), (M, N, K)
        assert torch.all(out[M] == 5.0) and torch.all(out[:, N] == 5.0), (M, N, K)
    assert seen == {0, 1, 2, 3}                       # every kernel of the file had its turn
    ops.check_device_errors()


@pytest.mark.parametrize("M,N,K,eps", [(1, 768, 768, 1e-5), (8, 2304, 768, 1e-5), (5, 1000, 96, 1e-6), (16, 320, 1600, 1e-5),
                                       (13, 50257, 64, 1e-3), (9, 200, 1024, 1e-5), (16, 4800, 2048, 1e-5),
                                       (8, 50257, 768, 1e-5), (11, 40000, 1600, 1e-5), (2, 50257, 1020, 1e-5)])
def test_stream_float32_product_with_the_norm_fused_in(ops, M, N, K, eps):
    """LayerNorm fused into the float32 weight-streaming product (the owning warp keeps the row in registers),
    also with gathered rows, against float64 and against the two separate kernels; one launch."""
    from mini_llm_b200.engine.context import Workspace
    ws = Workspace(torch.device(DEV), 64)
    x = rnd(M + 3, K, seed=1, scale=2.0) + 0.5
    gamma, beta = rnd(K, seed=2) + 1.0, rnd(K, seed=3)
    w, b = rnd(N, K, seed=4, scale=K ** -0.5), rnd(N, seed=5)
    for rows in (None, torch.tensor([(3 * i + 1) % (M + 3) for i in range(M)], dtype=torch.int32, device=DEV)):
        xin = x[:M] if rows is None else x
        src = xin.double() if rows is None else xin.double()[rows.long()]
        ref = torch.nn.functional.layer_norm(src, (K,), gamma.double(), beta.double(), eps) @ w.double().t() + b.double()
        for act in (None, "gelu_tanh"):
            want = ref if act is None else torch.nn.functional.gelu(ref, approximate="tanh")
            got = torch.full((M, N), 3.0, device=DEV)
            n0 = ops.launches
            ops.linear(ops.NormedInput(xin, gamma, beta, eps, rows, ws, torch.float32), w, b, out=got, act=act)
            assert ops.launches == n0 + 1
            assert (got.double() - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
        normed = torch.empty(M, K, device=DEV)
        ops.layernorm(xin, gamma, beta, eps, normed, rows=rows)
        two = torch.empty(M, N, device=DEV)
        ops.linear(normed, w, b, out=two, impl="stream_f32")
        got = torch.empty(M, N, device=DEV)
        ops.linear(ops.NormedInput(xin, gamma, beta, eps, rows, ws, torch.float32), w, b, out=got)
        assert (got.double() - two.double()).abs().max() < 2e-5 * max(1.0, ref.abs().max().item())
    # more than 16 rows or rows wider than 2048: the norm runs as a kernel of its own, the result is the same
    M2 = 20
    x2 = rnd(M2, K, seed=7)
    got = torch.empty(M2, N, device=DEV)
    ops.linear(ops.NormedInput(x2, gamma, beta, eps, None, ws, torch.float32), w, b, out=got)
    ref = torch.nn.functional.layer_norm(x2.double(), (K,), gamma.double(), beta.double(), eps) @ w.double().t() + b.double()
    assert (got.double() - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max().item())
    ops.check_device_errors()


@pytest.mark.parametrize("M,H,Hkv,dh,page,K", [(1, 12, 12, 64, 16, 768), (8, 4, 4, 16, 16, 64), (13, 3, 3, 32, 8, 96),
                                               (64, 6, 2, 64, 4, 128), (40, 25, 25, 64, 16, 1600)])
def test_stream_float32_qkv_product_writes_the_cache(ops, M, H, Hkv, dh, page, K):
    """The float32 Q|K|V projection whose epilogue puts keys and values into their page slots (with and without
    the fused norm), against the product followed by the copy kernel."""
    from mini_llm_b200.engine.context import Workspace
    ws = Workspace(torch.device(DEV), 64)
    q_size, kv = H * dh, Hkv * dh
    N = q_size + 2 * kv
    x = rnd(M, K, seed=1)
    w, b = rnd(N, K, seed=2, scale=K ** -0.5), rnd(N, seed=3)
    gamma, beta = rnd(K, seed=6) + 1.0, rnd(K, seed=7)
    P = 40
    g = torch.Generator().manual_seed(4)
    slots = torch.randperm(P * page, generator=g)[:M].to(torch.int32).to(DEV)
    for normed in (False, True):
        if normed:
            xin = torch.empty(M, K, device=DEV)
            ops.layernorm(x, gamma, beta, 1e-5, xin)
            arg = ops.NormedInput(x, gamma, beta, 1e-5, None, ws, torch.float32)
        else:
            xin = arg = x
        qkv = torch.empty(M, N, device=DEV)
        ops.linear(xin, w, b, out=qkv, impl="stream_f32")
        wk = torch.full((P, Hkv, page, dh), 9.0, device=DEV)
        wv = wk.clone()
        ops.kv_write(qkv[:, q_size:q_size + kv], qkv[:, q_size + kv:], wk, wv, slots)
        gk = torch.full((P, Hkv, page, dh), 9.0, device=DEV)
        gv = gk.clone()
        q_buf = torch.empty(M, q_size, device=DEV)
        n0 = ops.launches
        q = ops.linear_qkv_cache(arg, w, b, q_buf, gk, gv, slots, ws)
        assert ops.launches == n0 + (1 if (not normed or M <= 16) else 2)      # one launch; the norm apart beyond 16 rows
        assert q.data_ptr() == q_buf.data_ptr()
        tol = 0.0 if not normed or M > 16 else 2e-5 * max(1.0, qkv.abs().max().item())
        assert (q - qkv[:, :q_size]).abs().max() <= tol
        assert (gk - wk).abs().max() <= tol and (gv - wv).abs().max() <= tol
    ops.check_device_errors()


def test_linear_rows_do_not_depend_on_the_batch(ops):
    x, w = rnd(200, 96, seed=1), rnd(130, 96, seed=2)
    full = torch.empty(200, 130, device=DEV)
    ops.linear(x, w, None, out=full, impl="simt")
    for lo, hi in ((0, 1), (63, 65), (199, 200), (17, 150)):
        part = torch.empty(hi - lo, 130, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="simt")
        assert torch.equal(part, full[lo:hi])
    # the wide tiles used for many rows: same property
    x, w = rnd(700, 96, seed=3), rnd(260, 96, seed=4)
    full = torch.empty(700, 260, device=DEV)
    ops.linear(x, w, None, out=full, impl="simt")
    for lo, hi in ((0, 300), (129, 640), (400, 700)):
        part = torch.empty(hi - lo, 260, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="simt")
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("M,N,K", [(300, 768, 768), (2048, 768, 3072), (129, 1024, 1024), (400, 130, 3000)])
def test_linear_many_rows_float32_in_k_slices(ops, M, N, K):
    """The 32-bit product of many rows with a narrow result runs in K slices (chosen from N and K alone) whose partial
    sums a second kernel adds in slice order: against float64, with every epilogue, and a row's bits do not depend on
    how many rows are computed with it."""
    lib = ops.library()
    assert lib.mllm_linear_simt_splits(768, 768) > 1 and lib.mllm_linear_simt_splits(2304, 768) == 1
    x, w, b = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=K ** -0.5), rnd(N, seed=3)
    ref = x.double() @ w.double().t() + b.double()
    for act in (None, "gelu_tanh"):
        out = torch.full((M, N), 7.0, device=DEV)
        ops.linear(x, w, b, out=out, act=act, impl="simt")
        want = ref if act is None else torch.nn.functional.gelu(ref, approximate="tanh")
        assert (out.double() - want).abs().max() < 2e-5 * max(1.0, want.abs().max().item())
    acc = rnd(M, N, seed=4)
    acc0 = acc.clone()
    ops.linear(x, w, b, out=acc, accumulate=True, impl="simt")
    assert (acc.double() - (acc0.double() + ref)).abs().max() < 2e-5 * max(1.0, ref.abs().max().item())
    full = torch.empty(M, N, device=DEV)
    ops.linear(x, w, None, out=full, impl="simt")
    for lo, hi in ((0, 129), (M - 129, M), (max(0, M // 2 - 70), min(M, M // 2 + 70))):
        if hi - lo <= 128:
            continue                   # up to 128 rows another kernel (no slices) takes over: rounding may differ
        part = torch.empty(hi - lo, N, device=DEV)
        ops.linear(x[lo:hi], w, None, out=part, impl="simt")
        assert torch.equal(part, full[lo:hi]), (lo, hi)


def _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages, seed, sharp_key=None):
    """seqs: list of (context_len, q_len).  Returns everything the kernel needs plus dense K/V per sequence."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    k_pages = torch.zeros(num_pages, Hkv, page, dh)
    v_pages = torch.zeros(num_pages, Hkv, page, dh)
    tables, dense, token_seq, positions = [], [], [], []
    for s, (ctx, ql) in enumerate(seqs):
        n = (ctx + page - 1) // page
        tab = [perm.pop() for _ in range(n)]
        K = torch.randn(ctx, Hkv, dh, generator=g)
        V = torch.randn(ctx, Hkv, dh, generator=g)
        for p in range(ctx):
            k_pages[tab[p // page], :, p % page] = K[p]
            v_pages[tab[p // page], :, p % page] = V[p]
        tables.append(tab)
        dense.append((K, V))
        token_seq += [s] * ql
        positions += list(range(ctx - ql, ctx))
    T = len(token_seq)
    q = torch.randn(T, H * dh, generator=g)
    if sharp_key:
        # {sequence: [positions]}: every query of that sequence gets a common component that only the keys at
        # these positions answer (score about 36 at head size 64, against +-3 for the random keys), and each of
        # those keys has a value row of its own (2, 4, 6 ...), so that the result moves by O(1) when one of them
        # is dropped, or admitted where a window or the causal mask excludes it
        for s, where in sharp_key.items():
            u = torch.randn(Hkv, dh, generator=g)
            u = u / u.norm(dim=1, keepdim=True) * math.sqrt(dh)          # |u|^2 = dh for every head
            rows = [t for t, ts in enumerate(token_seq) if ts == s]
            uq = u.repeat_interleave(H // Hkv, dim=0).reshape(1, H * dh)
            q[rows] = q[rows] * 0.3 + uq * 1.5
            K, V = dense[s]
            for i, p in enumerate(where):
                K[p] = u * (24.0 / math.sqrt(dh))                        # (q.k)*dh^-0.5 = 1.5 * 24 = 36
                V[p] = 2.0 * (i + 1)
                k_pages[tables[s][p // page], :, p % page] = K[p]
                v_pages[tables[s][p // page], :, p % page] = V[p]
    mp = max(len(t) for t in tables)
    bt = torch.zeros(len(seqs), mp, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    return dict(q=q, k_pages=k_pages, v_pages=v_pages, bt=bt, token_seq=token_seq, positions=positions, dense=dense)


def _attention_reference(case, H, Hkv, dh, scale, window, dtype):
    q = case["q"].to(dtype).double()
    out = torch.zeros(q.shape[0], H * dh, dtype=torch.float64)
    for t, (s, p) in enumerate(zip(case["token_seq"], case["positions"])):
        K, V = case["dense"][s]
        K, V = K.to(dtype).double(), V.to(dtype).double()
        lo = max(0, p - window + 1) if window else 0
        for h in range(H):
            hk = h // (H // Hkv)
            sc = (K[lo:p + 1, hk] @ q[t, h * dh:(h + 1) * dh]) * scale
            out[t, h * dh:(h + 1) * dh] = torch.softmax(sc, 0) @ V[lo:p + 1, hk]
    return out


class _Ctx:
    pass


def _ctx_for(case):
    from mini_llm_b200.engine.context import Workspace
    ctx = _Ctx()
    ctx.token_seq = torch.tensor(case["token_seq"], dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor(case["positions"], dtype=torch.int32, device=DEV)
    ctx.ws = Workspace(torch.device(DEV), 64)
    ctx.max_ctx_len = max(case["positions"]) + 1
    ctx.decode_only = True
    return ctx


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,page,window", [(4, 4, 16, 16, None), (3, 3, 32, 8, None), (12, 12, 64, 16, None),
                                                  (6, 2, 64, 4, None), (2, 2, 128, 32, 300), (4, 1, 64, 16, 37),
                                                  (2, 1, 64, 24, 70), (2, 2, 32, 1, None)])
def test_decode_attention_split_keys(ops, dtype, H, Hkv, dh, page, window):
    """Single tokens at contexts around the split (128) and page edges, beside the plain kernel."""
    seqs = [(c, 1) for c in (1, 2, 16, 17, 127, 128, 129, 255, 256, 257, 513, 700, 1024)]
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=4096 // page + 24, seed=dh + page)
    ctx = _ctx_for(case)
    q = case["q"].to(dtype).to(DEV)
    kp, vp, bt = case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV)
    scale = dh ** -0.5
    out, plain = torch.empty_like(q), torch.empty_like(q)
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    ops.paged_attention(q, kp, vp, bt, ctx, out, impl="decode", **kw)
    ops.paged_attention(q, kp, vp, bt, ctx, plain, impl="simt", **kw)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - want).abs().max() < tol
    assert (out.double() - plain.double()).abs().max() < tol
    # the same splits merged through global scratch (the route of contexts beyond a cluster) give the same bits
    via_scratch = torch.empty_like(q)
    ops.paged_attention(q, kp, vp, bt, ctx, via_scratch, impl="decode_scratch", **kw)
    assert torch.equal(via_scratch, out)
    # a token's result does not depend on the tokens beside it
    one = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=4096 // page + 24, seed=dh + page)
    for t in (0, 5, 12):
        c1 = _Ctx()
        c1.token_seq, c1.positions = ctx.token_seq[t:t + 1].clone(), ctx.positions[t:t + 1].clone()
        c1.ws, c1.max_ctx_len, c1.decode_only = ctx.ws, int(ctx.positions[t]) + 1, True
        o1 = torch.empty_like(q[t:t + 1])
        ops.paged_attention(q[t:t + 1], kp, vp, bt, c1, o1, impl="decode", **kw)
        assert torch.equal(o1, out[t:t + 1])
        if dtype == torch.float32 and dh == 64:               # a small grid stages a split at a time
            assert ops.library().mllm_attention_decode_last_staging() == 1
    # nor on the size of the batch: with many tokens a CTA walks several splits (down to one CTA per token
    # and head), with few every split has its own CTA; the bits stay the same
    for reps in (4, 20):
        cb = _Ctx()
        cb.token_seq, cb.positions = ctx.token_seq.repeat(reps), ctx.positions.repeat(reps)
        cb.ws, cb.max_ctx_len, cb.decode_only = ctx.ws, ctx.max_ctx_len, True
        qb = q.repeat(reps, 1)
        ob = torch.empty_like(qb)
        ops.paged_attention(qb, kp, vp, bt, cb, ob, impl="decode", **kw)
        assert torch.equal(ob, out.repeat(reps, 1))
        if dtype == torch.float32 and dh == 64:               # a large one half a split at a time: the same bits
            assert ops.library().mllm_attention_decode_last_staging() == 2
        ops.paged_attention(qb, kp, vp, bt, cb, ob.zero_(), impl="decode_scratch", **kw)
        assert torch.equal(ob, out.repeat(reps, 1))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,page,window", [(4, 4, 16, 16, None), (3, 3, 32, 8, None), (6, 2, 64, 16, None),
                                                  (5, 1, 48, 4, None), (2, 2, 128, 32, 37), (2, 1, 256, 16, None)])
def test_paged_attention_mixed_batch(ops, dtype, H, Hkv, dh, page, window):
    seqs = [(1, 1), (70, 1), (33, 33), (100, 7), (16, 2), (129, 1)]       # first tokens, decodes, whole and partial prompts
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=128, seed=H * 100 + dh)
    # a far key that must dominate: query of the last sequence strongly matches its key at position 2
    K, V = case["dense"][5]
    t_last = len(case["token_seq"]) - 1
    scale = 1.0 / math.sqrt(dh)
    ctx = _Ctx()
    ctx.token_seq = torch.tensor(case["token_seq"], dtype=torch.int32, device=DEV)
    ctx.positions = torch.tensor(case["positions"], dtype=torch.int32, device=DEV)
    q = case["q"].to(dtype).to(DEV)
    out = torch.empty_like(q)
    ops.paged_attention(q, case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV), ctx,
                        out, num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert (out.double().cpu() - want).abs().max() < tol


@pytest.mark.parametrize("H,Hkv,dh,page,window", [(4, 4, 16, 16, None), (3, 3, 32, 8, None), (12, 12, 64, 16, None),
                                                  (6, 2, 64, 4, None), (2, 2, 128, 32, None), (4, 1, 64, 16, 37),
                                                  (2, 2, 64, 16, 100)])
def test_flash_attention_mixed_batch(ops, H, Hkv, dh, page, window):
    """Prompt portions of many lengths (tile edges at 64, page edges, portions that start in
    the middle of a key tile) beside single tokens, against float64 and the plain kernel."""
    from mini_llm_b200.engine.context import attention_tiles
    dtype = torch.bfloat16
    seqs = [(1, 1), (70, 1), (33, 33), (100, 7), (16, 2), (129, 129), (64, 64), (65, 65), (200, 63), (300, 130),
            (128, 64), (191, 2)]
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=1400 // page + 40, seed=H + dh + page)
    ctx = _ctx_for(case)
    ctx.decode_only = False
    tiles = attention_tiles([ql for _, ql in seqs])
    ctx.attn_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    ctx.n_tiles = len(tiles) // 3
    q = case["q"].to(dtype).to(DEV)
    kp, vp, bt = case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV)
    scale = dh ** -0.5
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    out, plain = torch.empty_like(q), torch.empty_like(q)
    ops.paged_attention(q, kp, vp, bt, ctx, out, impl="flash", **kw)
    ops.paged_attention(q, kp, vp, bt, ctx, plain, impl="simt", **kw)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    mag = want.abs().clamp(min=1.0)
    err = ((out.double().cpu() - want).abs() / mag).max(dim=1).values
    assert err.max() < 1e-2, (int(err.argmax()), float(err.max()))
    # two bfloat16 results that are each right to half a unit in the last place differ by at most one (2^-7 relative)
    assert ((out.double() - plain.double()).abs().cpu() / mag).max() < 2 ** -7 * 1.05
    # the same queries cut differently give the same bits
    seqs2 = [(129, 129)]
    c2 = _paged_case(dtype, seqs2, H, Hkv, dh, page, num_pages=1400 // page + 40, seed=99)
    ctxa = _ctx_for(c2)
    ctxa.decode_only = False
    ta = attention_tiles([129])
    ctxa.attn_tiles, ctxa.n_tiles = torch.tensor(ta, dtype=torch.int32, device=DEV), len(ta) // 3
    q2 = c2["q"].to(dtype).to(DEV)
    args2 = (c2["k_pages"].to(dtype).to(DEV), c2["v_pages"].to(dtype).to(DEV), c2["bt"].to(DEV))
    whole = torch.empty_like(q2)
    ops.paged_attention(q2, *args2, ctxa, whole, impl="flash", **kw)
    for lo, hi in ((0, 5), (5, 70), (70, 129), (100, 101)):
        cb = _Ctx()
        cb.token_seq = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
        cb.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        tb = attention_tiles([hi - lo])
        cb.attn_tiles, cb.n_tiles, cb.decode_only = torch.tensor(tb, dtype=torch.int32, device=DEV), len(tb) // 3, False
        part = torch.empty_like(q2[lo:hi])
        ops.paged_attention(q2[lo:hi], *args2, cb, part, impl="flash", **kw)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


@pytest.mark.parametrize("H,Hkv,page,window", [(2, 2, 16, None), (12, 12, 16, None), (6, 2, 8, None), (3, 1, 32, None),
                                               (2, 2, 128, None), (4, 1, 16, 37), (2, 2, 64, 200)])
def test_tcgen05_attention_mixed_batch(ops, H, Hkv, page, window):
    """The tensor-memory attention (128-query tiles, 128-key blocks, head size 64): prompt portions of
    many lengths (tile edges at 128, page edges, portions that start in the middle of a key block) beside
    single tokens, against float64 and the plain kernel; the same queries cut differently give the same bits."""
    from mini_llm_b200.engine.context import ATTN_TILE_WIDE, attention_tiles
    dtype, dh = torch.bfloat16, 64
    seqs = [(1, 1), (70, 1), (33, 33), (100, 7), (16, 2), (129, 129), (128, 128), (65, 65), (200, 63), (500, 300),
            (256, 128), (191, 2), (640, 257)]
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=2800 // page + 40, seed=H + page)
    ctx = _ctx_for(case)
    ctx.decode_only = False
    starts = [c - ql for c, ql in seqs]
    tiles = attention_tiles([ql for _, ql in seqs], starts, ATTN_TILE_WIDE)
    ctx.attn_tiles_wide = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    ctx.n_tiles_wide = len(tiles) // 3
    q = case["q"].to(dtype).to(DEV)
    kp, vp, bt = case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV)
    scale = dh ** -0.5
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    out, plain = torch.full_like(q, 7.0), torch.empty_like(q)
    ops.paged_attention(q, kp, vp, bt, ctx, out, impl="flash_tc", **kw)
    ops.check_device_errors()
    ops.paged_attention(q, kp, vp, bt, ctx, plain, impl="simt", **kw)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    mag = want.abs().clamp(min=1.0)
    err = ((out.double().cpu() - want).abs() / mag).max(dim=1).values
    assert err.max() < 1e-2, (int(err.argmax()), float(err.max()))
    assert ((out.double() - plain.double()).abs().cpu() / mag).max() < 2 ** -7 * 1.05
    # the same queries cut differently give the same bits
    c2 = _paged_case(dtype, [(300, 300)], H, Hkv, dh, page, num_pages=2800 // page + 40, seed=99)
    ctxa = _ctx_for(c2)
    ctxa.decode_only = False
    ta = attention_tiles([300], [0], ATTN_TILE_WIDE)
    ctxa.attn_tiles_wide, ctxa.n_tiles_wide = torch.tensor(ta, dtype=torch.int32, device=DEV), len(ta) // 3
    q2 = c2["q"].to(dtype).to(DEV)
    args2 = (c2["k_pages"].to(dtype).to(DEV), c2["v_pages"].to(dtype).to(DEV), c2["bt"].to(DEV))
    whole = torch.empty_like(q2)
    ops.paged_attention(q2, *args2, ctxa, whole, impl="flash_tc", **kw)
    for lo, hi in ((0, 5), (5, 70), (70, 300), (100, 101), (127, 260)):
        cb = _Ctx()
        cb.token_seq = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
        cb.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        tb = attention_tiles([hi - lo], [lo], ATTN_TILE_WIDE)
        cb.attn_tiles_wide, cb.n_tiles_wide, cb.decode_only = torch.tensor(tb, dtype=torch.int32, device=DEV), len(tb) // 3, False
        part = torch.empty_like(q2[lo:hi])
        ops.paged_attention(q2[lo:hi], *args2, cb, part, impl="flash_tc", **kw)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)
    ops.check_device_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,page,window", [(4, 4, 16, 16, None), (3, 3, 32, 8, None), (12, 12, 64, 16, None),
                                                  (5, 1, 48, 4, None), (2, 2, 128, 32, 100), (2, 1, 256, 16, None),
                                                  (4, 2, 80, 16, 37)])
def test_tiled_attention_mixed_batch(ops, dtype, H, Hkv, dh, page, window):
    """The CUDA-core tiled kernel (the 32-bit path's prefill attention, and head sizes such as 48 or
    80 on either path): prompt portions of many lengths beside single tokens, against float64 and
    the plain kernel; the same queries cut differently give the same bits."""
    from mini_llm_b200.engine.context import attention_tiles
    seqs = [(1, 1), (70, 1), (33, 33), (100, 7), (16, 2), (129, 129), (64, 64), (65, 65), (200, 63), (300, 130),
            (128, 64), (191, 2)]
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=1400 // page + 40, seed=H + dh + page)
    ctx = _ctx_for(case)
    ctx.decode_only = False
    tiles = attention_tiles([ql for _, ql in seqs])
    ctx.attn_tiles, ctx.n_tiles = torch.tensor(tiles, dtype=torch.int32, device=DEV), len(tiles) // 3
    q = case["q"].to(dtype).to(DEV)
    kp, vp, bt = case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV)
    scale = dh ** -0.5
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    out, plain = torch.empty_like(q), torch.empty_like(q)
    ops.paged_attention(q, kp, vp, bt, ctx, out, impl="tiled", **kw)
    ops.paged_attention(q, kp, vp, bt, ctx, plain, impl="simt", **kw)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    mag = want.abs().clamp(min=1.0)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -8
    assert ((out.double().cpu() - want).abs() / mag).max() < tol
    assert ((out.double() - plain.double()).abs().cpu() / mag).max() < (2e-5 if dtype == torch.float32 else 2 ** -7 * 1.05)
    c2 = _paged_case(dtype, [(129, 129)], H, Hkv, dh, page, num_pages=1400 // page + 40, seed=99)
    ctxa = _ctx_for(c2)
    ctxa.decode_only = False
    ta = attention_tiles([129])
    ctxa.attn_tiles, ctxa.n_tiles = torch.tensor(ta, dtype=torch.int32, device=DEV), len(ta) // 3
    q2 = c2["q"].to(dtype).to(DEV)
    args2 = (c2["k_pages"].to(dtype).to(DEV), c2["v_pages"].to(dtype).to(DEV), c2["bt"].to(DEV))
    whole = torch.empty_like(q2)
    ops.paged_attention(q2, *args2, ctxa, whole, impl="tiled", **kw)
    for lo, hi in ((0, 5), (5, 70), (70, 129), (100, 101)):
        cb = _Ctx()
        cb.token_seq = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
        cb.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        tb = attention_tiles([hi - lo])
        cb.attn_tiles, cb.n_tiles, cb.decode_only = torch.tensor(tb, dtype=torch.int32, device=DEV), len(tb) // 3, False
        part = torch.empty_like(q2[lo:hi])
        ops.paged_attention(q2[lo:hi], *args2, cb, part, impl="tiled", **kw)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,dh,page,window", [(2, 2, 64, 16, None), (12, 12, 64, 16, None), (6, 2, 32, 8, None), (3, 1, 48, 32, None),
                                                  (4, 4, 16, 4, None), (4, 1, 64, 16, 37), (2, 2, 64, 64, 200)])
def test_tiled_wide_attention_mixed_batch(ops, dtype, H, Hkv, dh, page, window):
    """The CUDA-core kernel with 128-query x 128-key tiles (the 32-bit path's attention for long prompt portions,
    heads of 16, 32, 48 and 64): portions of many lengths (tile edges at 128, page edges, portions that start in the
    middle of a key tile) beside single tokens, against float64 and the plain kernel; the same queries cut
    differently give the same bits."""
    from mini_llm_b200.engine.context import ATTN_TILE_WIDE, attention_tiles
    seqs = [(1, 1), (70, 1), (33, 33), (100, 7), (16, 2), (129, 129), (128, 128), (65, 65), (200, 63), (500, 300),
            (256, 128), (191, 2), (640, 257)]
    case = _paged_case(dtype, seqs, H, Hkv, dh, page, num_pages=2800 // page + 40, seed=H + page)
    ctx = _ctx_for(case)
    ctx.decode_only = False
    starts = [c - ql for c, ql in seqs]
    tiles = attention_tiles([ql for _, ql in seqs], starts, ATTN_TILE_WIDE)
    ctx.attn_tiles_wide = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    ctx.n_tiles_wide = len(tiles) // 3
    q = case["q"].to(dtype).to(DEV)
    kp, vp, bt = case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV)
    scale = dh ** -0.5
    kw = dict(num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=scale, window=window)
    out, plain = torch.full_like(q, 7.0), torch.empty_like(q)
    ops.paged_attention(q, kp, vp, bt, ctx, out, impl="tiled_wide", **kw)
    ops.paged_attention(q, kp, vp, bt, ctx, plain, impl="simt", **kw)
    want = _attention_reference(case, H, Hkv, dh, scale, window, dtype)
    mag = want.abs().clamp(min=1.0)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -8
    assert ((out.double().cpu() - want).abs() / mag).max() < tol
    assert ((out.double() - plain.double()).abs().cpu() / mag).max() < (2e-5 if dtype == torch.float32 else 2 ** -7 * 1.05)
    c2 = _paged_case(dtype, [(300, 300)], H, Hkv, dh, page, num_pages=2800 // page + 40, seed=99)
    ctxa = _ctx_for(c2)
    ctxa.decode_only = False
    ta = attention_tiles([300], [0], ATTN_TILE_WIDE)
    ctxa.attn_tiles_wide, ctxa.n_tiles_wide = torch.tensor(ta, dtype=torch.int32, device=DEV), len(ta) // 3
    q2 = c2["q"].to(dtype).to(DEV)
    args2 = (c2["k_pages"].to(dtype).to(DEV), c2["v_pages"].to(dtype).to(DEV), c2["bt"].to(DEV))
    whole = torch.empty_like(q2)
    ops.paged_attention(q2, *args2, ctxa, whole, impl="tiled_wide", **kw)
    for lo, hi in ((0, 5), (5, 70), (70, 300), (100, 101), (127, 260)):
        cb = _Ctx()
        cb.token_seq = torch.zeros(hi - lo, dtype=torch.int32, device=DEV)
        cb.positions = torch.arange(lo, hi, dtype=torch.int32, device=DEV)
        tb = attention_tiles([hi - lo], [lo], ATTN_TILE_WIDE)
        cb.attn_tiles_wide, cb.n_tiles_wide, cb.decode_only = torch.tensor(tb, dtype=torch.int32, device=DEV), len(tb) // 3, False
        part = torch.empty_like(q2[lo:hi])
        ops.paged_attention(q2[lo:hi], *args2, cb, part, impl="tiled_wide", **kw)
        assert torch.equal(part, whole[lo:hi]), (lo, hi)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """Random keys give near-uniform weights that would hide a skipped key; here one key
    far back carries almost all the weight, once at a page's first slot, once at its last."""
    H, dh, page = 2, 64, 16
    for far in (16 * 3, 16 * 3 + 15, 0, 299):
        case = _paged_case(dtype, [(300, 1)], H, H, dh, page, num_pages=32, seed=far)
        K, V = case["dense"][0]
        qv = case["q"][0].view(H, dh)
        K[far] = qv * 3.0                       # score ~ 3*|q|^2/sqrt(dh): dominates
        V[far] = 7.0
        tab = case["bt"][0].tolist()
        case["k_pages"][tab[far // page], :, far % page] = K[far]
        case["v_pages"][tab[far // page], :, far % page] = V[far]
        ctx = _ctx_for(case)
        q = case["q"].to(dtype).to(DEV)
        want = _attention_reference(case, H, H, dh, dh ** -0.5, None, dtype)
        for impl in ("simt", "decode"):
            out = torch.empty_like(q)
            ops.paged_attention(q, case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV),
                                case["bt"].to(DEV), ctx, out, num_heads=H, num_kv_heads=H, head_dim=dh,
                                scale=dh ** -0.5, impl=impl)
            assert (out.double().cpu() - want).abs().max() < (2e-5 if dtype == torch.float32 else 3e-2), impl
            assert out.float().mean().item() > 6.5, impl


@pytest.mark.parametrize("impl,dtype", [("tiled", torch.float32), ("tiled", torch.bfloat16), ("flash", torch.bfloat16),
                                        ("flash_tc", torch.bfloat16), ("tiled_wide", torch.float32),
                                        ("tiled_wide", torch.bfloat16)])
def test_prompt_attention_finds_one_far_key_among_hundreds(ops, impl, dtype):
    """The same for the kernels of prompt portions: the last 150 queries of a 700-token request all lean on one
    key far back - at a page's first and last slot, in the first key tile, at a tile's edge - which sits in
    another key tile or block than the queries; a kernel that skipped or misplaced that tile shows at once."""
    from mini_llm_b200.engine.context import ATTN_TILE_WIDE, attention_tiles
    H, dh, page, ctx_len, ql = 2, 64, 16, 700, 150
    for far in (0, 16 * 3 + 15, 127, 128, 383, 549):
        case = _paged_case(dtype, [(ctx_len, ql)], H, H, dh, page, num_pages=64, seed=far)
        K, V = case["dense"][0]
        u = torch.randn(H, dh, generator=torch.Generator().manual_seed(far + 1))
        case["q"] = (case["q"].view(ql, H, dh) * 0.3 + u * 1.5).reshape(ql, H * dh)   # all queries get a common component ...
        K[far] = u * 3.0                                        # ... that one key answers: its score is about 36
        V[far] = 7.0
        tab = case["bt"][0].tolist()
        case["k_pages"][tab[far // page], :, far % page] = K[far]
        case["v_pages"][tab[far // page], :, far % page] = V[far]
        ctx = _ctx_for(case)
        ctx.decode_only = False
        t64 = attention_tiles([ql], [ctx_len - ql])
        t128 = attention_tiles([ql], [ctx_len - ql], ATTN_TILE_WIDE)
        ctx.attn_tiles, ctx.n_tiles = torch.tensor(t64, dtype=torch.int32, device=DEV), len(t64) // 3
        ctx.attn_tiles_wide, ctx.n_tiles_wide = torch.tensor(t128, dtype=torch.int32, device=DEV), len(t128) // 3
        q = case["q"].to(dtype).to(DEV)
        want = _attention_reference(case, H, H, dh, dh ** -0.5, None, dtype)
        out = torch.empty_like(q)
        ops.paged_attention(q, case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV),
                            ctx, out, num_heads=H, num_kv_heads=H, head_dim=dh, scale=dh ** -0.5, impl=impl)
        assert (out.double().cpu() - want).abs().max() < (2e-5 * 8 if dtype == torch.float32 else 3e-2), (impl, far)
        assert out.float().mean().item() > 6.0, (impl, far)
    ops.check_device_errors()


@pytest.mark.parametrize("window", [None, 200])
@pytest.mark.parametrize("impl,dtype", [("simt", torch.float32), ("decode", torch.float32), ("decode", torch.bfloat16),
                                        ("tiled", torch.float32), ("tiled", torch.bfloat16), ("flash", torch.bfloat16),
                                        ("flash_tc", torch.bfloat16), ("tiled_wide", torch.float32)])
def test_attention_edges_with_sharp_keys(ops, impl, dtype, window):
    """Keys that carry the weight sit exactly where an off-by-one would drop or admit them: position 0, the
    first and last key of a page and of a 128-key block, the query's own position, and with a window its first
    key (p - window + 1, seen) and the key just outside it (p - window, not seen).  Every such key has a value row
    of its own, so one wrong decision moves the result by O(1), far above any rounding."""
    from mini_llm_b200.engine.context import ATTN_TILE_WIDE, attention_tiles
    H, Hkv, dh, page, ctx_len = 4, 2, 64, 16, 700
    ql = 1 if impl in ("decode", "simt") else 150
    last = ctx_len - 1
    for trial in range(3):
        if window is None:
            where = [[0, 15, 16, last], [127, 128, last - 1], [383, 384, 640, 0]][trial]
        else:
            # for the last query: its window's first key and the one before it; for earlier queries of a portion
            # the same pair moves with them, so keys all along the edge are placed
            where = [[last - window + 1, last - window, last], [last - window, 511, 512],
                     [last - ql + 1 - window + 1, last - ql + 1 - window, 639, 640]][trial]
            where = [p for p in where if p >= 0]
        case = _paged_case(dtype, [(40, 1 if ql == 1 else 7), (ctx_len, ql)], H, Hkv, dh, page, num_pages=64,
                           seed=trial, sharp_key={1: where})
        ctx = _ctx_for(case)
        ctx.decode_only = ql == 1
        qls, starts = [1 if ql == 1 else 7, ql], [40 - (1 if ql == 1 else 7), ctx_len - ql]
        t64 = attention_tiles(qls, starts)
        t128 = attention_tiles(qls, starts, ATTN_TILE_WIDE)
        ctx.attn_tiles, ctx.n_tiles = torch.tensor(t64, dtype=torch.int32, device=DEV), len(t64) // 3
        ctx.attn_tiles_wide, ctx.n_tiles_wide = torch.tensor(t128, dtype=torch.int32, device=DEV), len(t128) // 3
        q = case["q"].to(dtype).to(DEV)
        want = _attention_reference(case, H, Hkv, dh, dh ** -0.5, window, dtype)
        out = torch.empty_like(q)
        ops.paged_attention(q, case["k_pages"].to(dtype).to(DEV), case["v_pages"].to(dtype).to(DEV), case["bt"].to(DEV),
                            ctx, out, num_heads=H, num_kv_heads=Hkv, head_dim=dh, scale=dh ** -0.5, window=window,
                            impl=impl)
        err = ((out.double().cpu() - want).abs() / want.abs().clamp(min=1.0)).max()
        assert err < (2e-4 if dtype == torch.float32 else 1e-2), (impl, window, trial, float(err))
        # the test has teeth: dropping the first sharp key from the reference moves it by far more than that
        K, V = case["dense"][1]
        V[where[0]] += 5.0
        moved = (_attention_reference(case, H, Hkv, dh, dh ** -0.5, window, dtype) - want).abs().max()
        assert moved > 0.5 or (window is not None and where[0] == last - window), (trial, float(moved))
    ops.check_device_errors()


def test_resolve_tokens(ops):
    """Ids that stand for "row r of the last sampling launch" (negative) are filled in on the device."""
    ids = torch.tensor([5, -1, 17, -3, -2, 0, -4], dtype=torch.int32, device=DEV)
    sampled = torch.tensor([100, 200, 300, 400], dtype=torch.int32, device=DEV)
    ops.resolve_tokens(ids, sampled)
    assert ids.tolist() == [5, 100, 17, 300, 200, 0, 400]


def test_paged_attention_refuses_sizes_it_cannot_take(ops):
    from mini_llm_b200.ops import KernelError
    ctx = _Ctx()
    ctx.token_seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx.positions = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dh in (8, 24, 272):
        q = torch.zeros(1, 2 * dh, device=DEV)
        pages = torch.zeros(2, 2, 4, dh, device=DEV)
        with pytest.raises(KernelError):
            ops.paged_attention(q, pages, pages, torch.zeros(1, 1, dtype=torch.int32, device=DEV), ctx,
                                torch.empty_like(q), num_heads=2, num_kv_heads=2, head_dim=dh, scale=1.0)
    with pytest.raises(KernelError):
        ops.linear(torch.zeros(2, 4), torch.zeros(3, 4), None, out=torch.zeros(2, 3))      # CPU tensors: no CPU path


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_write(ops, dtype):
    T, Hkv, dh, page, P = 37, 3, 32, 8, 11
    qkv = rnd(T, 5 * Hkv * dh, seed=1, dtype=dtype)
    k, v = qkv[:, Hkv * dh:2 * Hkv * dh], qkv[:, 3 * Hkv * dh:4 * Hkv * dh]
    g = torch.Generator().manual_seed(2)
    slots = torch.randperm(P * page, generator=g)[:T].to(torch.int32).to(DEV)
    kp = torch.zeros(P, Hkv, page, dh, device=DEV, dtype=dtype)
    vp = torch.zeros_like(kp)
    ops.kv_write(k, v, kp, vp, slots)
    wk, wv = torch.zeros_like(kp), torch.zeros_like(vp)
    for t in range(T):
        s = int(slots[t])
        wk[s // page, :, s % page] = k[t].view(Hkv, dh)
        wv[s // page, :, s % page] = v[t].view(Hkv, dh)
    assert torch.equal(kp, wk) and torch.equal(vp, wv)


@pytest.mark.parametrize("R,V", [(1, 17), (5, 1000), (64, 50257), (3, 1025), (8, 50257), (1, 151936), (2, 8192)])
def test_argmax_and_sampling(ops, R, V):
    logits = rnd(R, V, seed=R + V, scale=3.0)
    logits[0, 3] = logits[0, min(9, V - 1)] = logits[0].max() + 1          # equal maxima: the lowest id wins
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    want = torch.tensor([int((row == row.max()).nonzero()[0, 0]) for row in logits.cpu()], dtype=torch.int32)
    assert torch.equal(out.cpu(), want)
    g = torch.Generator().manual_seed(5)
    for temp in (0.8, 1.7):
        u = torch.rand(R, generator=g)
        temps = torch.full((R,), temp)
        temps[R // 2] = 0.0                                              # greedy rows beside sampled ones
        ops.sample(logits, temps.to(DEV), u.to(DEV), out)
        got = out.cpu()
        for r in range(R):
            if temps[r] == 0:
                assert got[r] == want[r]
                continue
            p = torch.softmax(logits[r].double().cpu() / temp, 0)
            c = torch.cumsum(p, 0)
            exact = int((c > u[r].double()).nonzero()[0, 0]) if (c > u[r].double()).any() else V - 1
            if got[r] != exact:                                         # only where u sits on an edge of the CDF
                edge = min(abs(float(c[exact]) - float(u[r])), abs(float(c[exact - 1]) - float(u[r])) if exact else 1.0)
                assert edge < 1e-5, (r, int(got[r]), exact, edge)
    # the distribution itself: many draws from one row
    row = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]]).repeat(4000, 1).to(DEV)
    u = torch.rand(4000, generator=g).to(DEV)
    o = torch.empty(4000, dtype=torch.int32, device=DEV)
    ops.sample(row, torch.ones(4000, device=DEV), u, o)
    freq = torch.bincount(o.cpu().long(), minlength=5).double() / 4000
    assert (freq - torch.softmax(row[0].double().cpu(), 0)).abs().max() < 0.03


def test_a_kernel_that_gives_up_is_noticed_by_the_host(ops):
    """Kernels with bounded waits write a pinned host word when a wait runs out; the host reads it for free
    wherever it has waited for the stream.  Here a one-thread kernel writes the word the same way (no wait
    is made to run out)."""
    ops.library()
    torch.cuda.synchronize()
    ops.raise_if_kernel_gave_up()            # nothing so far
    ops._call("mllm_debug_report_error", 203, ops._stream())
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="tcgen05 attention.*code 3"):
        ops.raise_if_kernel_gave_up()
    ops.raise_if_kernel_gave_up()            # reported once
    ops._call("mllm_debug_report_error", 301, ops._stream())
    with pytest.raises(ops.KernelError, match="decode attention"):
        ops.check_device_errors()            # the thorough check synchronises by itself
    ops.check_device_errors()
