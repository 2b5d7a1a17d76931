"""The decode attention entry point that brings its own scratch memory.

mllm_attention_decode_noalloc is meant for callers that cannot allocate device memory when
they call (memory owned by another component of their process, a point in their program
where cudaMalloc is not allowed or would stall the device).  The test calls the exported C
symbol through ctypes, as such a caller would, twice in a row with different inputs, and
compares each result, bit for bit, with what the ordinary entry point gives for the same
inputs on the same route; the second call also shows that what the first left in the shared
scratch does no harm.  The
file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, T, H, dh, page, dtype):
    g = torch.Generator().manual_seed(seed)
    ctx_lens = torch.randint(1, 900, (T,), generator=g).tolist()
    ctx_lens[0], ctx_lens[-1] = 1, 1024
    pages_per = [(c + page - 1) // page for c in ctx_lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    k_pages = torch.randn(n_pages, H, page, dh, generator=g).to(dtype).to(DEV)
    v_pages = torch.randn(n_pages, H, page, dh, generator=g).to(dtype).to(DEV)
    bt = torch.zeros(T, max(pages_per), dtype=torch.int32)
    for s, n in enumerate(pages_per):
        bt[s, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    q = torch.randn(T, H * dh, generator=g).to(dtype).to(DEV)
    token_seq = torch.arange(T, dtype=torch.int32, device=DEV)
    positions = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=DEV)
    return q, k_pages, v_pages, bt.to(DEV), token_seq, positions, max(ctx_lens)


@pytest.mark.parametrize("dtype,dcode", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_no_alloc_entry_point_matches_the_ordinary_one(dtype, dcode):
    from mini_llm_b200 import ops
    from mini_llm_b200.csrc import build
    from mini_llm_b200.engine.context import Workspace

    ops.library()
    lib = ctypes.CDLL(build.library_path())                     # the exported C symbol, as a C caller sees it
    fn = lib.mllm_attention_decode_noalloc
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, ll, vp, vp, vp, ci, vp, vp, vp, ll, ci, ci, ci, ci, ci, cf, ci, ci, ci, vp]
    fn.restype = ci
    lib.mllm_last_error.restype = ctypes.c_char_p
    H, dh, page = 12, 64, 16
    stream = torch.cuda.current_stream().cuda_stream
    for call, (seed, T) in enumerate([(1, 8), (2, 5)]):         # two calls in a row
        q, kp, vpg, bt, token_seq, positions, max_ctx = _case(seed, T, H, dh, page, dtype)
        max_splits = ops.decode_splits(max_ctx)
        got = torch.empty_like(q)
        rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vpg.data_ptr(), bt.data_ptr(), bt.stride(0),
                token_seq.data_ptr(), positions.data_ptr(), got.data_ptr(), got.stride(0), T, H, H, dh, page,
                dh ** -0.5, 0, max_splits, dcode, stream)
        assert rc == 0, lib.mllm_last_error().decode()

        class Ctx:
            pass
        ctx = Ctx()
        ctx.token_seq, ctx.positions, ctx.max_ctx_len, ctx.decode_only = token_seq, positions, max_ctx, True
        ctx.ws = Workspace(torch.device(DEV), 64)
        want = torch.empty_like(q)
        # the ordinary entry point on the same route (splits meet in global scratch): the same kernel with the
        # same partial results in the same merge order, so the two outputs must be equal bit for bit; a fault
        # in how the built-in scratch is carved up or cleared cannot hide inside a tolerance
        ops.paged_attention(q, kp, vpg, bt, ctx, want, num_heads=H, num_kv_heads=H, head_dim=dh, scale=dh ** -0.5,
                            impl="decode_scratch")
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), f"call {call}: max difference {(got.double() - want.double()).abs().max()}"
        # and within the kernel tests' tolerance of the route that generation takes (splits meet in a cluster)
        ops.paged_attention(q, kp, vpg, bt, ctx, want, num_heads=H, num_kv_heads=H, head_dim=dh, scale=dh ** -0.5,
                            impl="decode")
        torch.cuda.synchronize()
        tol = 2e-5 if dtype == torch.float32 else 1e-2
        assert (got.double() - want.double()).abs().max() < tol, f"call {call}"
    # sizes beyond the built-in scratch are refused, with a reason, and nothing runs
    rc = fn(q.data_ptr(), q.stride(0), kp.data_ptr(), vpg.data_ptr(), bt.data_ptr(), bt.stride(0),
            token_seq.data_ptr(), positions.data_ptr(), got.data_ptr(), got.stride(0), 64, 32, 32, dh, page,
            dh ** -0.5, 0, 8, dcode, stream)
    assert rc != 0 and b"exceeds the built-in scratch" in lib.mllm_last_error()
