"""The kernel library: the Python face of the CUDA sources in ``csrc/``.

Every function checks its arguments (device, dtype, layout, sizes the kernel can
take) and then calls one exported C function with raw device pointers and the
current CUDA stream.  There is no CPU fallback and no library attention or model
code behind these names: if the shared library cannot be built or loaded, or a
tensor is not on a CUDA device, the call fails with an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
SMALL_M = 64                 # rows up to which the weight-streaming product is used
SMALL_M_F32 = 64             # the same for the float32 weight-streaming product (csrc/linear_stream_f32.cu)
NORM_FUSE_M_F32 = 16         # rows up to which that product takes the norm into its loads (rows up to 2048 wide)
DECODE_SPLIT = 128           # keys per split of the decode attention (csrc/attention_decode.cu)
DECODE_CLUSTER_SPLITS = 8    # splits that can meet in one thread-block cluster (MAX_CLUSTER there)
_FLASH_HEAD_DIMS = (16, 32, 64, 128)
_DECODE_HEAD_DIMS = {torch.bfloat16: (16, 32, 64, 128, 256), torch.float32: (16, 32, 64, 128)}
_ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_erf": 2}
_lib = None

c_int, c_ll, c_float, c_void_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


def _signatures(lib):
    lib.mllm_last_error.restype = ctypes.c_char_p
    lib.mllm_abi_version.restype = c_int
    lib.mllm_set_pdl.argtypes = [c_int]
    lib.mllm_set_pdl.restype = c_int
    sig = {
        "mllm_embed": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "mllm_resolve_tokens": [c_void_p, c_int, c_void_p, c_int, c_void_p],
        "mllm_layernorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_kv_write": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                          c_void_p],
        "mllm_linear_simt": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_void_p, c_ll, c_void_p],
        "mllm_linear_simt_splits": [c_int, c_int],
        "mllm_attention_simt": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                c_ll, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_linear_smallm": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_void_p],
        "mllm_linear_smallm_fused": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_linear_stream_f32": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_int, c_int, c_void_p],
        "mllm_linear_stream_f32_tall_rows": [c_int, c_int],
        "mllm_linear_stream_f32_kernel_of": [c_int, c_int, c_int],
        "mllm_linear_stream_f32_bind_error": [c_void_p],
        "mllm_linear_stream_f32_error": [c_void_p],
        "mllm_linear_tcgen05": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p],
        "mllm_linear_tcgen05_qkv": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "mllm_tcgen05_error": [c_void_p],
        "mllm_tcgen05_bind_error": [c_void_p],
        "mllm_attention_tcgen05_bind_error": [c_void_p],
        "mllm_attention_decode_bind_error": [c_void_p],
        "mllm_debug_report_error": [c_int, c_void_p],
        "mllm_attention_decode": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_int, c_int, c_int, c_void_p],
        "mllm_attention_decode_last_staging": [],
        "mllm_attention_flash": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                 c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_attention_tcgen05": [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "mllm_attention_tcgen05_error": [c_void_p],
        "mllm_attention_decode_error": [c_void_p],
        "mllm_attention_tiled": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                 c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_attention_tiled_wide": [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                      c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "mllm_argmax": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p],
        "mllm_argmax_sliced": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "mllm_sample": [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


def library():
    """The loaded shared library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.ensure_built()
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from e
        _signatures(lib)
        _lib = lib
        _bind_error_word(lib)
    return _lib


_error_word = None      # one int32 in pinned host memory: kernels that give up on a bounded wait write it


def _bind_error_word(lib) -> None:
    """Give the kernels that have bounded waits the address of a pinned host word (a no-op
    without a CUDA device: the library can be built and loaded on a machine that has none)."""
    global _error_word
    if _error_word is not None or not torch.cuda.is_available():
        return
    word = torch.zeros(1, dtype=torch.int32).pin_memory()
    for name in ("mllm_tcgen05_bind_error", "mllm_attention_tcgen05_bind_error", "mllm_attention_decode_bind_error",
                 "mllm_linear_stream_f32_bind_error"):
        if getattr(lib, name)(word.data_ptr()) != 0:
            raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    _error_word = word


_WHO = {1: "the tcgen05 product", 2: "the tcgen05 attention", 3: "the decode attention",
        4: "the float32 weight-streaming product"}


def raise_if_kernel_gave_up() -> None:
    """Costs one read of host memory: call it wherever the host has just waited for the
    stream (after tokens or logits were fetched).  Raises once per event."""
    if _error_word is None:
        return
    code = int(_error_word[0])
    if code:
        _error_word[0] = 0
        raise KernelError(f"{_WHO.get(code // 100, 'a kernel')} gave up on a bounded wait (code {code % 100}): "
                          "the results of the step are not valid")


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for the kernels that support it: the next kernel's
    blocks may start (and prefetch weights) while the current kernel drains."""
    library().mllm_set_pdl(int(bool(on)))


def is_loaded() -> bool:
    return _lib is not None


launches = 0       # kernels launched through this module (bench.py reports the count)


_timeline = None    # a list while time_launches() is active: (entry point, start event, end event) per launch


def _call(name: str, *args) -> None:
    global launches
    lib = library()
    launches += 1
    if _timeline is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = getattr(lib, name)(*args)
        e1.record()
        _timeline.append((name, e0, e1))
    else:
        rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name}: {lib.mllm_last_error().decode(errors='replace')}")


class time_launches:
    """Times every launch made inside the scope with a pair of CUDA events (eager launches only: nothing can be
    recorded inside a graph capture).  ``rows()`` afterwards gives (entry point, launches, total ms) per entry
    point in order of first use: the per-kernel share of a step, in the manner of the reference's stage timer
    (include/profiling/stage_timer.cuh:40-101), without a device synchronisation per stage."""

    def __enter__(self):
        global _timeline
        self._old, _timeline = _timeline, []
        self._mine = _timeline
        return self

    def __exit__(self, *a):
        global _timeline
        _timeline = self._old

    def rows(self):
        torch.cuda.synchronize()
        agg = {}
        for name, e0, e1 in self._mine:
            n, ms = agg.get(name, (0, 0.0))
            agg[name] = (n + 1, ms + e0.elapsed_time(e1))
        return [(k, n, ms) for k, (n, ms) in agg.items()]


def check_device_errors() -> None:
    """Raise if a kernel gave up on a bounded wait since the last check.  Synchronises and reads
    the kernels' own device words (the thorough check of tests and tools; the engine uses
    raise_if_kernel_gave_up, which costs nothing)."""
    code = c_int(0)
    lib = library()
    torch.cuda.synchronize()
    raise_if_kernel_gave_up()
    if lib.mllm_tcgen05_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        who = {1: "the TMA producer (no free stage)", 2: "the MMA issuer (no full stage)",
               3: "the epilogue (accumulator never ready)"}.get(code.value, "?")
        raise KernelError(f"a tcgen05 kernel gave up waiting: code {code.value}, {who}")
    if lib.mllm_attention_tcgen05_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError(f"the tcgen05 attention kernel gave up waiting: code {code.value} "
                          "(1 producer, 2-6 MMA issuer, 7-8 softmax warps)")
    if lib.mllm_attention_decode_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError("the decode attention kernel gave up waiting for a split's keys and values")
    if lib.mllm_linear_stream_f32_error(ctypes.byref(code)) != 0:
        raise KernelError(lib.mllm_last_error().decode(errors="replace"))
    if code.value:
        raise KernelError("the float32 weight-streaming product gave up waiting for its weights")


_stream_handle = None     # set by stream_scope(); None: ask torch on every call


class stream_scope:
    """Within the scope every launch goes to the stream that is current on entry, without
    asking torch again on each call (a lookup costs more than the launch itself)."""

    def __enter__(self):
        global _stream_handle
        self._old = _stream_handle
        _stream_handle = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *a):
        global _stream_handle
        _stream_handle = self._old


def _stream() -> int:
    return _stream_handle if _stream_handle is not None else torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16")


def _cuda(name: str, t: torch.Tensor, dtype=None, contiguous=True):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _rows(name: str, t: torch.Tensor):
    """A 2-D tensor whose rows are contiguous; returns its row stride in elements."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


# --------------------------------------------------------------------------- embedding
def embed(ids, positions, table, pos_table, out) -> None:
    """out[t] = table[ids[t]] (+ pos_table[positions[t]]), 32-bit."""
    _cuda("ids", ids, torch.int32)
    _cuda("table", table)
    _cuda("out", out, torch.float32)
    T, D = out.shape
    if ids.numel() != T or table.shape[1] != D:
        raise KernelError(f"embed: {ids.numel()} ids, table {tuple(table.shape)}, out {tuple(out.shape)}")
    pp = None
    if pos_table is not None:
        _cuda("positions", positions, torch.int32)
        _cuda("pos_table", pos_table, table.dtype)
        if pos_table.shape[1] != D or positions.numel() != T:
            raise KernelError("embed: position table or positions do not fit")
        pp = pos_table.data_ptr()
    _call("mllm_embed", ids.data_ptr(), positions.data_ptr() if pos_table is not None else None,
          table.data_ptr(), pp, out.data_ptr(), T, D, _dt(table), _stream())


def resolve_tokens(ids, sampled) -> None:
    """In place: ids[t] = sampled[-ids[t] - 1] wherever ids[t] is negative (a token that the
    last sampling launch left on the device and the host has not read yet)."""
    _cuda("ids", ids, torch.int32)
    _cuda("sampled", sampled, torch.int32)
    _call("mllm_resolve_tokens", ids.data_ptr(), ids.numel(), sampled.data_ptr(), sampled.numel(), _stream())


# --------------------------------------------------------------------------- norm
def layernorm(x, gamma, beta, eps: float, out, rows=None) -> None:
    """out[r] = LayerNorm(x[rows[r]] or x[r]); x 32-bit, out 32-bit or bfloat16."""
    _cuda("x", x, torch.float32)
    _cuda("gamma", gamma, torch.float32)
    _cuda("beta", beta, torch.float32)
    _cuda("out", out)
    D = x.shape[1]
    R = out.shape[0]
    if gamma.numel() != D or beta.numel() != D or out.shape[1] != D:
        raise KernelError(f"layernorm: width {D} against gamma {gamma.numel()}, out {tuple(out.shape)}")
    if rows is not None:
        _cuda("rows", rows, torch.int32)
        if rows.numel() != R:
            raise KernelError("layernorm: rows and out differ in length")
    elif x.shape[0] != R:
        raise KernelError("layernorm: x and out differ in rows")
    _call("mllm_layernorm", x.data_ptr(), rows.data_ptr() if rows is not None else None, gamma.data_ptr(),
          beta.data_ptr(), out.data_ptr(), R, D, float(eps), _dt(out), _stream())


# --------------------------------------------------------------------------- linear
class NormedInput:
    """LayerNorm(x[rows]) not yet computed: a product that can fuse the norm into its
    loads takes it as it is, anything else calls ``materialize()``."""

    def __init__(self, x, gamma, beta, eps, rows, ws, dtype):
        self.x, self.gamma, self.beta, self.eps, self.rows, self.ws, self.dtype = x, gamma, beta, eps, rows, ws, dtype
        self.shape = (x.shape[0] if rows is None else rows.shape[0], x.shape[1])
        self._out = None

    def materialize(self):
        if self._out is None:
            out = self.ws.buf("norm_out", self.shape[0], self.shape[1], self.dtype)
            layernorm(self.x, self.gamma, self.beta, self.eps, out, rows=self.rows)
            self._out = out
        return self._out


def decode_splits(max_ctx_len: int) -> int:
    """Key splits the decode attention is launched with: just enough for the longest context
    (launching more costs: the splits of a request form a cluster that is scheduled as a whole)."""
    return max(1, -(-int(max_ctx_len) // DECODE_SPLIT))


_sm_count = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _sm_count


def _small_m_wins(M: int, N: int, K: int) -> bool:
    """Whether the weight-streaming kernel (mma.sync, 16 weight rows per CTA, K split over its warps) beats the
    tensor-memory kernel for M rows of bfloat16.  Measured in replayed graphs at the shapes of GPT-2 small, medium
    and XL (N = D, 3D, 4D and K = D, 4D for D = 768, 1024, 1600, and the 50,257-row head): up to 16 rows the
    streaming kernel needs one pass of its token tiles and wins everywhere (2.3-12 us against 6-27 us), except
    that a matrix as tall as a vocabulary is streamed faster by the tensor-memory kernel from 9 rows on; from 17
    to 32 rows it makes two passes and still wins while its N/16 CTAs fit the SMs in one wave (N <= 2368 on 148
    SMs: 4.4 against 5.7 us at N = 2304, 8.1 against 5.8 us at N = 3072); beyond 32 rows it loses everywhere (it
    reads its input rows from L2 again and again while the other stays near its fixed cost)."""
    if M <= 8:
        return True
    if N >= 16384:
        return False
    if M <= 16:
        return True
    if M <= 32:
        return -(-N // 16) <= sm_count()
    return False


def _fusable(weight, M, K) -> bool:
    return weight.dtype == torch.bfloat16 and M <= SMALL_M and K % 8 == 0 and weight.data_ptr() % 16 == 0


NORM_FUSE_M = 16             # rows up to which the norm is recomputed inside every CTA of the product


def _norm_ok(n: NormedInput) -> bool:
    x = n.x
    return (n.shape[0] <= NORM_FUSE_M and x.dtype == torch.float32 and x.stride(1) == 1 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0
            and n.gamma.data_ptr() % 16 == 0 and n.beta.data_ptr() % 16 == 0)


def _linear_fused(x, weight, bias, out, act, accumulate, norm: Optional[NormedInput], kv) -> None:
    """The small-M product with the norm fused on its input and/or the cache write on its output."""
    M = norm.shape[0] if norm is not None else x.shape[0]
    N, K = weight.shape
    ldo = _rows("out", out)
    if norm is not None:
        xp, ldx = None, norm.x.stride(0)
        nargs = (norm.x.data_ptr(), norm.rows.data_ptr() if norm.rows is not None else None,
                 norm.gamma.data_ptr(), norm.beta.data_ptr(), float(norm.eps))
    else:
        xp, ldx = x.data_ptr(), _rows("x", x)
        nargs = (None, None, None, None, 0.0)
    if kv is not None:
        k_pages, v_pages, slots, q_size = kv
        _, Hkv, ps, dh = k_pages.shape
        kargs = (k_pages.data_ptr(), v_pages.data_ptr(), slots.data_ptr(), int(q_size), Hkv, dh, ps)
    else:
        kargs = (None, None, None, 0, 0, 0, 0)
    _call("mllm_linear_smallm_fused", xp, ldx, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), _dt(out), *nargs, *kargs, _stream())


STREAM_F32_MAX_K = 12288      # the longest rows whose tiles fit the streaming product's shared memory in every case


def _stream_f32_ok(weight, M, K) -> bool:
    return (weight.dtype == torch.float32 and M <= SMALL_M_F32 and K % 4 == 0 and K <= STREAM_F32_MAX_K
            and weight.data_ptr() % 16 == 0)


def _norm_ok_f32(n: NormedInput) -> bool:
    x = n.x
    return (n.shape[0] <= NORM_FUSE_M_F32 and n.shape[1] <= 2048 and x.dtype == torch.float32 and x.stride(1) == 1
            and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and n.gamma.data_ptr() % 16 == 0
            and n.beta.data_ptr() % 16 == 0)


def _linear_stream_f32(x, weight, bias, out, act, accumulate, norm: Optional[NormedInput], kv) -> None:
    """The float32 weight-streaming product, with the norm fused on its input and/or the cache write on its output."""
    M = norm.shape[0] if norm is not None else x.shape[0]
    N, K = weight.shape
    ldo = _rows("out", out)
    if norm is not None:
        xp, ldx = None, norm.x.stride(0)
        nargs = (norm.x.data_ptr(), norm.rows.data_ptr() if norm.rows is not None else None,
                 norm.gamma.data_ptr(), norm.beta.data_ptr(), float(norm.eps))
    else:
        xp, ldx = x.data_ptr(), _rows("x", x)
        nargs = (None, None, None, None, 0.0)
    if kv is not None:
        k_pages, v_pages, slots, q_size = kv
        _, Hkv, ps, dh = k_pages.shape
        kargs = (k_pages.data_ptr(), v_pages.data_ptr(), slots.data_ptr(), int(q_size), Hkv, dh, ps)
    else:
        kargs = (None, None, None, 0, 0, 0, 0)
    _call("mllm_linear_stream_f32", xp, ldx, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), *nargs, *kargs, _stream())


def linear_qkv_cache(x, weight, bias, q_out, k_pages, v_pages, slot_mapping, ws):
    """Q|K|V projection whose keys and values go to their page slots; returns the queries.

    weight [q_size + 2*kv_heads*head_dim, K]; q_out [M, q_size] is where the queries may be
    put.  The cache write rides in the product's epilogue - the weight-streaming kernel's with few
    rows (which also takes a NormedInput's norm into its loads), the tensor-memory kernel's with
    many - and q_out is returned; where neither applies (32-bit, head sizes that are no multiple
    of 32) the product writes a [M, N] buffer, kv_write copies keys and values from it, and the
    buffer's query columns are returned.
    """
    M = x.shape[0]
    N, K = weight.shape
    q_size = q_out.shape[1]
    _, Hkv, ps, dh = k_pages.shape
    if N != q_size + 2 * Hkv * dh:
        raise KernelError(f"linear_qkv_cache: {N} output columns against {q_size} + 2*{Hkv}*{dh}")
    _cuda("q_out", q_out, contiguous=False)
    _cuda("k_pages", k_pages, q_out.dtype)
    _cuda("v_pages", v_pages, q_out.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    if slot_mapping.numel() != M or q_out.shape[0] != M or v_pages.shape != k_pages.shape:
        raise KernelError(f"linear_qkv_cache: {M} rows, {slot_mapping.numel()} slots, q_out {tuple(q_out.shape)}")
    norm = x if isinstance(x, NormedInput) else None
    if q_out.dtype == torch.float32 and _stream_f32_ok(weight, M, K) and q_out.stride(1) == 1 \
            and k_pages.is_contiguous() and v_pages.is_contiguous():
        # float32, few rows: the weight-streaming product writes keys and values from its epilogue
        if norm is not None and not _norm_ok_f32(norm):
            x, norm = norm.materialize(), None
        if norm is not None or (x.is_cuda and x.dtype == torch.float32 and _rows("x", x) % 4 == 0 and x.data_ptr() % 16 == 0):
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            _linear_stream_f32(None if norm is not None else x, weight, bias, q_out, None, False, norm,
                               (k_pages, v_pages, slot_mapping, q_size))
            return q_out
    if norm is not None and not _norm_ok(norm):
        x, norm = norm.materialize(), None
    if q_out.dtype == torch.bfloat16 and _fusable(weight, M, K) and _small_m_wins(M, N, K) and (
            _norm_ok(norm) if norm is not None else
            (x.is_cuda and x.dtype == torch.bfloat16 and _rows("x", x) % 8 == 0 and x.data_ptr() % 16 == 0)):
        if bias is not None:
            _cuda("bias", bias, torch.float32)
        _linear_fused(None if norm is not None else x, weight, bias, q_out, None, False, norm,
                      (k_pages, v_pages, slot_mapping, q_size))
        return q_out
    if norm is not None:
        x, norm = norm.materialize(), None
    _cuda("x", x, contiguous=False)
    if (q_out.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and not _small_m_wins(M, N, K) and q_size % 32 == 0 and dh % 32 == 0 and K % 8 == 0
            and _rows("x", x) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and _rows("q_out", q_out) % 8 == 0 and q_out.data_ptr() % 16 == 0 and k_pages.is_contiguous()
            and v_pages.is_contiguous()):
        # many rows: the tensor-memory product, whose epilogue stores keys and values into their pages
        if bias is not None:
            _cuda("bias", bias, torch.float32)
        _call("mllm_linear_tcgen05_qkv", x.data_ptr(), _rows("x", x), weight.data_ptr(),
              bias.data_ptr() if bias is not None else None, q_out.data_ptr(), _rows("q_out", q_out), M, N, K,
              k_pages.data_ptr(), v_pages.data_ptr(), slot_mapping.data_ptr(), q_size, Hkv, dh, ps, _stream())
        return q_out
    qkv = ws.buf("qkv", M, N, q_out.dtype)
    linear(x, weight, bias, out=qkv)
    kv_write(qkv[:, q_size:q_size + Hkv * dh], qkv[:, q_size + Hkv * dh:], k_pages, v_pages, slot_mapping)
    return qkv[:, :q_size]


def linear(x, weight, bias, out, act: Optional[str] = None, accumulate: bool = False, impl: Optional[str] = None):
    """out = act(x @ weight^T + bias) (+ out when ``accumulate``).

    x [M,K] rows contiguous (a column slice is fine) or a NormedInput, weight [N,K]
    contiguous, bias [N] 32-bit or None, out [M,N] rows contiguous.  float32 operands run
    the true 32-bit FMA kernel; bfloat16 operands accumulate in 32-bit.
    """
    if isinstance(x, NormedInput):
        if impl in (None, "smallm") and _fusable(weight, x.shape[0], weight.shape[1]) and _norm_ok(x) \
                and (impl == "smallm" or _small_m_wins(x.shape[0], weight.shape[0], weight.shape[1])) \
                and x.shape[1] == weight.shape[1] and tuple(out.shape) == (x.shape[0], weight.shape[0]):
            _cuda("out", out, contiguous=False)
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            if act not in _ACT:
                raise KernelError(f"linear: unknown activation {act!r}")
            _linear_fused(None, weight, bias, out, act, accumulate, x, None)
            return out
        if impl in (None, "stream_f32") and _stream_f32_ok(weight, x.shape[0], weight.shape[1]) and _norm_ok_f32(x) \
                and out.dtype == torch.float32 and x.shape[1] == weight.shape[1] \
                and tuple(out.shape) == (x.shape[0], weight.shape[0]):
            _cuda("out", out, contiguous=False)
            if bias is not None:
                _cuda("bias", bias, torch.float32)
            if act not in _ACT:
                raise KernelError(f"linear: unknown activation {act!r}")
            _linear_stream_f32(None, weight, bias, out, act, accumulate, x, None)
            return out
        x = x.materialize()
    _cuda("x", x, contiguous=False)
    _cuda("weight", weight, x.dtype)
    _cuda("out", out, contiguous=False)
    lda = _rows("x", x)
    ldo = _rows("out", out)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"linear: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _cuda("bias", bias, torch.float32)
        if bias.numel() != N:
            raise KernelError("linear: bias length")
    if act not in _ACT:
        raise KernelError(f"linear: unknown activation {act!r}")
    if x.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("linear: float32 operands need a float32 result")
    if impl is None:
        impl = "simt"
        if x.dtype == torch.bfloat16 and K % 8 == 0 and lda % 8 == 0 \
                and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
            impl = "smallm" if _small_m_wins(M, N, K) else "tcgen05"
        elif x.dtype == torch.float32 and out.dtype == torch.float32 and _stream_f32_ok(weight, M, K) \
                and lda % 4 == 0 and x.data_ptr() % 16 == 0:
            impl = "stream_f32"
    if impl == "stream_f32":
        _linear_stream_f32(x, weight, bias, out, act, accumulate, None, None)
        return out
    if impl in ("smallm", "tcgen05"):
        _call("mllm_linear_" + impl, x.data_ptr(), lda, weight.data_ptr(),
              bias.data_ptr() if bias is not None else None, out.data_ptr(), ldo, M, N, K, _ACT[act],
              int(accumulate), _dt(out), _stream())
        return out
    if impl != "simt":
        raise KernelError(f"linear: unknown implementation {impl!r}")
    ws_ptr, ws_floats = None, 0
    if x.dtype == torch.float32 and M > 128:
        # many rows in 32-bit: a narrow result is computed in K slices whose partial sums need room
        splits = library().mllm_linear_simt_splits(N, K)
        if splits > 1:
            ws = _scratch("simt_splitk", x.device, splits * M * N)
            ws_ptr, ws_floats = ws.data_ptr(), ws.numel()
    _call("mllm_linear_simt", x.data_ptr(), lda, weight.data_ptr(), bias.data_ptr() if bias is not None else None,
          out.data_ptr(), ldo, M, N, K, _ACT[act], int(accumulate), _dt(x), _dt(out), ws_ptr, ws_floats, _stream())
    if ws_ptr is not None:
        global launches
        launches += 1           # the finishing kernel that adds the slices
    return out


_scratch_bufs = {}


def _scratch(name: str, device, floats: int) -> torch.Tensor:
    """A float32 scratch buffer of this module that only grows (a step shape runs eagerly before it is captured as a
    graph, so a captured graph never sees the buffer replaced under it unless a larger shape comes later: sizes are
    rounded up to the next power of two to make that rare, and the runner drops its graphs when it happens)."""
    global scratch_version
    key = (name, str(device))
    buf = _scratch_bufs.get(key)
    if buf is None or buf.numel() < floats:
        buf = torch.empty(max(1 << (int(floats) - 1).bit_length(), 1 << 20), dtype=torch.float32, device=device)
        _scratch_bufs[key] = buf
        scratch_version += 1
    return buf


scratch_version = 0     # bumped whenever a scratch buffer of this module is replaced


# --------------------------------------------------------------------------- cache
def kv_write(k, v, k_pages, v_pages, slot_mapping) -> None:
    """Copy rows of k and v ([T, kv_heads*head_dim], same row stride) to their slots."""
    _cuda("k", k, contiguous=False)
    _cuda("v", v, k.dtype, contiguous=False)
    _cuda("k_pages", k_pages, k.dtype)
    _cuda("v_pages", v_pages, k.dtype)
    _cuda("slot_mapping", slot_mapping, torch.int32)
    ld = _rows("k", k)
    if _rows("v", v) != ld:
        raise KernelError("kv_write: k and v differ in row stride")
    _, Hkv, ps, dh = k_pages.shape
    T = k.shape[0]
    if k.shape[1] != Hkv * dh or slot_mapping.numel() != T or v_pages.shape != k_pages.shape:
        raise KernelError("kv_write: shapes do not fit the pages")
    _call("mllm_kv_write", k.data_ptr(), v.data_ptr(), ld, k_pages.data_ptr(), v_pages.data_ptr(),
          slot_mapping.data_ptr(), T, Hkv, dh, ps, _dt(k), _stream())


attention_launches = {}     # attention kernel name -> launches so far (tests check which kernel a step took)
use_tcgen05_attention = True    # False: prompt portions stay on the mma.sync kernel (for comparisons and profiles)


def _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo) -> bool:
    return (q.dtype == torch.bfloat16 and head_dim == 64 and 8 <= ps <= 128 and ps & (ps - 1) == 0
            and getattr(ctx, "n_tiles_wide", 0) > 0 and ldq % 8 == 0 and q.data_ptr() % 16 == 0 and ldo % 8 == 0
            and out.data_ptr() % 16 == 0 and k_pages.is_contiguous() and k_pages.data_ptr() % 16 == 0)


_TILED_WIDE_HEAD_DIMS = (16, 32, 48, 64)


def _tiled_wide_ok(q, head_dim, ctx, ldq) -> bool:
    """Long prompt portions (128-row tiles mostly full) with heads up to 64, where no tensor-core kernel applies."""
    nw = getattr(ctx, "n_tiles_wide", 0)
    return (head_dim in _TILED_WIDE_HEAD_DIMS and nw > 0 and ctx.T >= 256 and ctx.T >= 80 * nw
            and ldq % (16 // q.element_size()) == 0 and q.data_ptr() % 16 == 0)


def paged_attention(q, k_pages, v_pages, block_table, ctx, out, *, num_heads, num_kv_heads, head_dim, scale,
                    window=None, impl: Optional[str] = None) -> None:
    """Causal attention of the step's tokens over the cache.

    q [T, heads*head_dim] (rows contiguous), pages [num_pages, kv_heads, page_size,
    head_dim], block_table [S, max_pages] int32, ctx.token_seq / ctx.positions [T].
    """
    _cuda("q", q, contiguous=False)
    _cuda("k_pages", k_pages, q.dtype)
    _cuda("v_pages", v_pages, q.dtype)
    _cuda("out", out, q.dtype, contiguous=False)
    _cuda("block_table", block_table, torch.int32, contiguous=False)
    ldq = _rows("q", q)
    ldo = _rows("out", out)
    T = q.shape[0]
    _, Hkv, ps, dh = k_pages.shape
    if Hkv != num_kv_heads or dh != head_dim or q.shape[1] != num_heads * head_dim:
        raise KernelError("paged_attention: head counts or sizes do not fit the pages")
    if head_dim % 16 != 0 or not (16 <= head_dim <= 256):
        raise KernelError(f"paged_attention: head size {head_dim} is not a multiple of 16 in 16..256")
    bt_stride = _rows("block_table", block_table)
    if impl is None:
        impl = "simt"
        if getattr(ctx, "decode_only", False) and head_dim in _DECODE_HEAD_DIMS[q.dtype] and ldq % 8 == 0 \
                and q.data_ptr() % 16 == 0:
            impl = "decode"
        elif use_tcgen05_attention and _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo) and ctx.T >= 256 \
                and ctx.T >= 80 * ctx.n_tiles_wide:
            impl = "flash_tc"       # long prompt portions (tiles of 128 rows mostly full): the tensor-memory kernel
        elif q.dtype == torch.bfloat16 and head_dim in _FLASH_HEAD_DIMS and getattr(ctx, "n_tiles", 0) > 0 \
                and ldq % 8 == 0 and q.data_ptr() % 16 == 0 and ldo % 2 == 0:
            impl = "flash"
        elif _tiled_wide_ok(q, head_dim, ctx, ldq):
            impl = "tiled_wide"     # float32 (or a head size of 48) and long portions: 128 x 128 tiles on CUDA cores
        elif getattr(ctx, "n_tiles", 0) > 0:
            impl = "tiled"          # float32, or a head size the tensor-core kernel does not take
    attention_launches[impl] = attention_launches.get(impl, 0) + 1
    if impl == "tiled_wide":
        if head_dim not in _TILED_WIDE_HEAD_DIMS or getattr(ctx, "n_tiles_wide", 0) <= 0 or ldq % (16 // q.element_size()):
            raise KernelError("paged_attention: the 128 x 128 CUDA-core kernel takes head sizes "
                              f"{_TILED_WIDE_HEAD_DIMS}, 16-byte aligned rows and a list of 128-row tiles")
        _call("mllm_attention_tiled_wide", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles_wide.data_ptr(), int(ctx.n_tiles_wide),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _dt(q), _stream())
        return
    if impl == "tiled":
        _call("mllm_attention_tiled", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles.data_ptr(), int(ctx.n_tiles),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _dt(q), _stream())
        return
    if impl == "flash_tc":
        if not _flash_tc_ok(q, k_pages, out, ctx, head_dim, ps, ldq, ldo):
            raise KernelError("paged_attention: the tcgen05 kernel takes bfloat16, head size 64, pages of 8..128 "
                              "tokens (a power of two), 16-byte aligned rows and a list of 128-row tiles")
        _call("mllm_attention_tcgen05", q.data_ptr(), ldq, T, k_pages.data_ptr(), v_pages.data_ptr(),
              int(k_pages.shape[0]), block_table.data_ptr(), bt_stride, ctx.attn_tiles_wide.data_ptr(),
              int(ctx.n_tiles_wide), ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim,
              ps, float(scale), int(window or 0), _stream())
        return
    if impl == "flash":
        if q.dtype != torch.bfloat16 or head_dim not in _FLASH_HEAD_DIMS:
            raise KernelError(f"paged_attention: the tensor-core kernel takes bfloat16 and head sizes "
                              f"{_FLASH_HEAD_DIMS}, not {q.dtype} / {head_dim}")
        _call("mllm_attention_flash", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.attn_tiles.data_ptr(), int(ctx.n_tiles),
              ctx.positions.data_ptr(), out.data_ptr(), ldo, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), _stream())
        return
    if impl in ("decode", "decode_scratch"):        # "decode_scratch": splits meet in global scratch, not in a cluster
        if head_dim not in _DECODE_HEAD_DIMS[q.dtype]:
            raise KernelError(f"paged_attention: the split-key kernel takes head sizes {_DECODE_HEAD_DIMS[q.dtype]} "
                              f"for {q.dtype}, not {head_dim}")
        # splits cover the longest context of the step, rounded up so that captured graphs keep their grid
        max_splits = decode_splits(ctx.max_ctx_len)
        # Up to DECODE_CLUSTER_SPLITS splits meet in a thread-block cluster and touch no scratch; only beyond that
        # (contexts over 1,024 tokens) or on request do the partial results go through global memory.  Asking for
        # the buffers only then keeps a growing context from ever replacing a buffer under the captured graphs.
        if impl == "decode_scratch" or max_splits > DECODE_CLUSTER_SPLITS:
            part_o = ctx.ws.buf("attn_part_o", T * num_heads * max_splits, head_dim, torch.float32).data_ptr()
            part_ml = ctx.ws.buf("attn_part_ml", T * num_heads * max_splits, 2, torch.float32).data_ptr()
            counters = ctx.ws.zeroed("attn_counters", T * num_heads).data_ptr()     # the kernel leaves them zero
        else:
            part_o = part_ml = counters = None
        _call("mllm_attention_decode", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(),
              block_table.data_ptr(), bt_stride, ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(),
              ldo, part_o, part_ml, counters, T, num_heads, num_kv_heads, head_dim, ps, float(scale),
              int(window or 0), max_splits, _dt(q), int(impl == "decode_scratch"), _stream())
        return
    if impl != "simt":
        raise KernelError(f"paged_attention: unknown implementation {impl!r}")
    _call("mllm_attention_simt", q.data_ptr(), ldq, k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
          bt_stride, ctx.token_seq.data_ptr(), ctx.positions.data_ptr(), out.data_ptr(), ldo, T, num_heads,
          num_kv_heads, head_dim, ps, float(scale), int(window or 0), _dt(q), _stream())


# --------------------------------------------------------------------------- sampling
_argmax_scratch = {}


def argmax(logits, out) -> None:
    """out[r] = index of the largest value of row r, the lowest index among equals."""
    _cuda("logits", logits, torch.float32, contiguous=False)
    _cuda("out", out, torch.int32)
    ld = _rows("logits", logits)
    R, V = logits.shape
    if out.numel() != R:
        raise KernelError("argmax: one output per row")
    slices = 1
    if R * 4 < 592 and V >= 8192:            # few long rows: cut them so that the SMs have work
        slices = min(64, max(2, 592 // max(R, 1)), V // 1024)
    if slices == 1:
        _call("mllm_argmax", logits.data_ptr(), ld, R, V, out.data_ptr(), _stream())
        return
    dev = logits.device
    sc = _argmax_scratch.get(dev)
    if sc is None or sc[0].numel() < R * slices or sc[2].numel() < R:
        n = max(R * slices, 4096)
        sc = (torch.empty(n, dtype=torch.float32, device=dev), torch.empty(n, dtype=torch.int32, device=dev),
              torch.zeros(max(R, 1024), dtype=torch.int32, device=dev))
        _argmax_scratch[dev] = sc
    _call("mllm_argmax_sliced", logits.data_ptr(), ld, R, V, out.data_ptr(), sc[0].data_ptr(), sc[1].data_ptr(),
          sc[2].data_ptr(), slices, _stream())


def sample(logits, temperature, uniform, out) -> None:
    """Per row: argmax if temperature == 0, else an inverse-CDF draw with uniform[r]."""
    _cuda("logits", logits, torch.float32, contiguous=False)
    _cuda("temperature", temperature, torch.float32)
    _cuda("uniform", uniform, torch.float32)
    _cuda("out", out, torch.int32)
    ld = _rows("logits", logits)
    R, V = logits.shape
    if temperature.numel() != R or uniform.numel() != R or out.numel() != R:
        raise KernelError("sample: per-row arguments differ in length")
    _call("mllm_sample", logits.data_ptr(), ld, R, V, temperature.data_ptr(), uniform.data_ptr(), out.data_ptr(),
          _stream())
