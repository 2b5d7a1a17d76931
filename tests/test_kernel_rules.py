"""Which float32 weight-streaming kernel takes which shape: the rules of csrc/linear_stream_f32.cu, read through the
library without a GPU (they depend on the matrix, on the side of a row count and on the number of SMs, for which the
library assumes a B200's 148 when it finds no device).  The reference has one small-M kernel chosen for M < 4 and four
shapes (src/kernels/decode_gemm.cu:171-210); here the choice is a measured rule, and this test pins what it says for
the layer shapes of GPT-2 small, medium and XL."""
import ctypes

import pytest

FEW, MANY, TALL, LONG = 0, 1, 2, 3


@pytest.fixture(scope="module")
def lib():
    from mini_llm_b200.csrc import build

    lib = ctypes.CDLL(build.ensure_built())
    for name in ("mllm_linear_stream_f32_kernel_of",):
        getattr(lib, name).argtypes = [ctypes.c_int] * 3
    lib.mllm_linear_stream_f32_tall_rows.argtypes = [ctypes.c_int] * 2
    try:
        import torch
        if torch.cuda.is_available() and torch.cuda.get_device_properties(0).multi_processor_count != 148:
            pytest.skip("the pinned choices are those of a GPU with 148 SMs")
    except ImportError:
        pass
    return lib


def kernel(lib, M, N, K):
    return lib.mllm_linear_stream_f32_kernel_of(M, N, K)


@pytest.mark.parametrize("D,F", [(768, 3072), (1024, 4096), (1600, 6400)])
def test_decode_projections_of_gpt2_sizes(lib, D, F):
    V = 50257
    for M in (1, 8, 16):
        assert kernel(lib, M, 3 * D, D) == TALL          # Q|K|V
        assert kernel(lib, M, F, D) == TALL              # up-projection
        assert kernel(lib, M, V, D) == TALL              # the head
    # the output projection: narrow and, at XL's width, longer than 1024: the tile kernel's K slices win there
    assert kernel(lib, 8, D, D) == (TALL if D <= 1024 else FEW)
    # the down-projection: cluster slices where their chunks fill the slice, else the tile kernel up to 16 rows
    assert kernel(lib, 8, D, F) == (FEW if D == 1024 else LONG)
    assert kernel(lib, 40, D, F) == LONG
    # the vocabulary takes every row count that fits shared memory
    assert lib.mllm_linear_stream_f32_tall_rows(V, D) == {768: 64, 1024: 48, 1600: 32}[D]
    assert kernel(lib, 64, V, D) == (TALL if D == 768 else MANY)


def test_row_counts_beyond_the_registers_kernel(lib):
    # 2304 x 768: up to 16 rows; 3072 x 768 (tiles of 32 rows fill more than half of the SMs): up to 48; 4800 x 1600: up to 24
    assert lib.mllm_linear_stream_f32_tall_rows(2304, 768) == 16
    assert lib.mllm_linear_stream_f32_tall_rows(3072, 768) == 48
    assert lib.mllm_linear_stream_f32_tall_rows(4800, 1600) == 24
    assert lib.mllm_linear_stream_f32_tall_rows(1600, 1600) == 0
    assert kernel(lib, 17, 2304, 768) == MANY and kernel(lib, 48, 3072, 768) == TALL and kernel(lib, 49, 3072, 768) == MANY
    # rows longer than 2048 never go to the registers kernel, whatever their number
    assert lib.mllm_linear_stream_f32_tall_rows(50257, 2052) == 0
    # a kernel is named for every row count up to 64
    for M in range(1, 65):
        assert kernel(lib, M, 1000, 96) in (FEW, MANY, TALL, LONG)
