// Split-key decode attention without any buffer from the caller besides inputs and output.
//
// This entry point has no counterpart in the reference (taejuk/mini-llm allocates all its
// scratch with cudaMalloc when its model object is built, src/model/gpt2_model.cu:178-205).
//
// Who needs it.  mllm_attention_decode() wants three scratch buffers from its caller.  Some
// callers have no way to get device memory when they call: a host program that links this
// library into a process whose GPU memory is owned and carved up by another component (a
// rendering engine, another framework's pool, a fixed real-time partition) and that may not
// call cudaMalloc at all; code that runs at a point where an allocation is forbidden or
// would stall everything, since cudaMalloc and cudaFree synchronise the whole device; and
// plain C callers without an allocator of their own.  For them the scratch lives inside the
// library, in a file-scope device array of fixed size.
//
// The price and the limits:
//   * every GPU that loads the library gives up the array's
//     MLLM_NOALLOC_MAX_SLOTS * (MLLM_NOALLOC_MAX_HEAD_DIM + 3) * 4 bytes (about 4.1 MB)
//     from the moment the library is loaded until the process ends, used or not;
//   * a call needs tokens x heads x max_splits <= MLLM_NOALLOC_MAX_SLOTS and a head size
//     <= MLLM_NOALLOC_MAX_HEAD_DIM; anything larger is refused with an error (return value
//     1, text from mllm_last_error()), nothing is launched;
//   * all calls share the one array.  Two calls that may run on the GPU at the same time
//     (different streams, or different host threads without ordering between them) race on
//     it and give wrong results: order them on one stream or with events;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
//     stream capture;
//   * it calls no cudaMalloc, cudaFree or allocating library routine.  It clears the
//     counters it needs with one cudaMemsetAsync on the caller's stream and then launches
//     the same kernel as mllm_attention_decode().
//
// Arguments are those of mllm_attention_decode() without part_o, part_ml and counters:
//   q [T, H*dh] (row stride q_stride elements), k_pages/v_pages [pages, Hkv, page_size, dh],
//   block_table [requests, bt_stride] int32, token_seq/positions [T] int32 (the request of
//   every token and its absolute position), out [T, H*dh] (row stride out_stride),
//   scale, window (0 = all keys), max_splits, dtype 0 = float32, 1 = bfloat16, stream.
// The caller guarantees max_splits >= ceil((largest position + 1) / 128): the positions are
// on the device, so this cannot be checked here, and a token that needs more splits gets no
// output written.  Everything the host can check is checked before anything is launched:
// null pointers, heads, page size > 0, window >= 0, block table stride > 0, and that q (with
// its row stride) and the two pools are 16-byte aligned.
// Returns 0, or a non-zero code with the reason in mllm_last_error().
#pragma once
#include <cuda_runtime.h>

#define MLLM_NOALLOC_MAX_SLOTS 8192
#define MLLM_NOALLOC_MAX_HEAD_DIM 128

#ifdef __cplusplus
extern "C" {
#endif

int mllm_attention_decode_noalloc(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                  const int* block_table, int bt_stride, const int* token_seq, const int* positions,
                                  void* out, long long out_stride, int T, int H, int Hkv, int dh, int page_size,
                                  float scale, int window, int max_splits, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
