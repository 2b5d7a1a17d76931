"""The decode attention's C entry points refuse what a raw C caller can get wrong (sizes, null
pointers, alignment) on the host, before any CUDA call: these checks run on a machine without a
GPU, and on one with a GPU nothing is launched.  Pointers here are made-up addresses that are
never dereferenced, because every call must be refused first."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    from mini_llm_b200.csrc import build

    lib = ctypes.CDLL(build.ensure_built())
    lib.mllm_last_error.restype = ctypes.c_char_p
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    lib.mllm_attention_decode_noalloc.argtypes = [vp, ll, vp, vp, vp, ci, vp, vp, vp, ll, ci, ci, ci, ci, ci, cf, ci, ci, ci, vp]
    lib.mllm_attention_decode_noalloc.restype = ci
    lib.mllm_attention_decode.argtypes = [vp, ll, vp, vp, vp, ci, vp, vp, vp, ll, vp, vp, vp, ci, ci, ci, ci, ci, cf,
                                          ci, ci, ci, ci, vp]
    lib.mllm_attention_decode.restype = ci
    return lib


GOOD = dict(q=0x10000, q_stride=768, k=0x20000, v=0x30000, bt=0x40000, bt_stride=64, seq=0x50000, pos=0x60000,
            out=0x70000, out_stride=768, T=4, H=12, Hkv=12, dh=64, page=16, scale=0.125, window=0, splits=4, dtype=1)


def _noalloc(lib, **kw):
    a = dict(GOOD, **kw)
    rc = lib.mllm_attention_decode_noalloc(a["q"], a["q_stride"], a["k"], a["v"], a["bt"], a["bt_stride"], a["seq"], a["pos"],
                                           a["out"], a["out_stride"], a["T"], a["H"], a["Hkv"], a["dh"], a["page"],
                                           a["scale"], a["window"], a["splits"], a["dtype"], None)
    return rc, lib.mllm_last_error().decode()


def _plain(lib, **kw):
    a = dict(GOOD, **kw)
    rc = lib.mllm_attention_decode(a["q"], a["q_stride"], a["k"], a["v"], a["bt"], a["bt_stride"], a["seq"], a["pos"],
                                   a["out"], a["out_stride"], a.get("part_o"), a.get("part_ml"), a.get("counters"),
                                   a["T"], a["H"], a["Hkv"], a["dh"], a["page"], a["scale"], a["window"], a["splits"],
                                   a["dtype"], a.get("scratch_only", 0), None)
    return rc, lib.mllm_last_error().decode()


BAD = [
    (dict(page=0), "page size 0"),
    (dict(page=-16), "page size"),
    (dict(window=-1), "window -1"),
    (dict(bt_stride=0), "row stride 0"),
    (dict(k=0x20008), "16-byte aligned"),
    (dict(v=0x30004), "16-byte aligned"),
    (dict(q=0x10002), "queries must be 16-byte aligned"),
    (dict(q_stride=770), "queries must be 16-byte aligned"),
    (dict(q=None), "null pointer"),
    (dict(pos=None), "null pointer"),
    (dict(out=None), "null pointer"),
    (dict(Hkv=5), "12 heads over 5"),
    (dict(Hkv=0), "heads"),
    (dict(dh=48), "head size 48"),
    (dict(dtype=7), "dtype code 7"),
    (dict(dtype=0, dh=256), "head size 256"),
]


@pytest.mark.parametrize("change,text", BAD, ids=[t for _, t in BAD])
def test_bad_arguments_are_refused_before_any_launch(lib, change, text):
    for call in (_noalloc, _plain):
        rc, msg = call(lib, **change)
        assert rc == 1 and text in msg, (call.__name__, rc, msg)


def test_sizes_beyond_the_built_in_scratch_are_refused(lib):
    rc, msg = _noalloc(lib, T=64, H=32, Hkv=32, splits=8)
    assert rc == 1 and "exceeds the built-in scratch" in msg
    rc, msg = _noalloc(lib, splits=0)
    assert rc == 1


def test_many_splits_need_the_callers_scratch(lib):
    rc, msg = _plain(lib, splits=9)
    assert rc == 1 and "need the scratch buffers" in msg
    rc, msg = _plain(lib, splits=4, scratch_only=1)
    assert rc == 1 and "need the scratch buffers" in msg


def test_no_tokens_is_nothing_to_do(lib):
    assert _noalloc(lib, T=0, page=0)[0] == 0
    assert _plain(lib, T=0, q=None)[0] == 0
