// Token embedding gather with the additive position table fused in:
// x[t,:] = table[id_t,:] (+ pos_table[pos_t,:]), written as 32-bit.
// Same arithmetic as the reference's embedding_kernel (src/kernels/embedding.cu:23-43),
// for any width and either table dtype; row offsets are 64-bit.
#include "common.cuh"

template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const int* __restrict__ pos,
                             const T* __restrict__ table, const T* __restrict__ pos_table,
                             float* __restrict__ out, int D) {
    const int t = blockIdx.x;
    pdl_launch();               // the first kernel of a step: nothing before it to wait for
    const T* row = table + (size_t)ids[t] * D;
    const T* prow = pos_table ? pos_table + (size_t)pos[t] * D : nullptr;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = to_f32(row[d]);
        if (prow) v += to_f32(prow[d]);
        o[d] = v;
    }
}

MLLM_EXPORT int mllm_embed(const int* ids, const int* pos, const void* table, const void* pos_table,
                           float* out, int T, int D, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D <= 0) return mllm_fail(1, "embed: width %d", D);
    int threads = D >= 256 ? 256 : ((D + 31) / 32) * 32;
    if (dtype == MLLM_F32)
        embed_kernel<float><<<T, threads, 0, stream>>>(ids, pos, (const float*)table, (const float*)pos_table, out, D);
    else if (dtype == MLLM_BF16)
        embed_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(ids, pos, (const __nv_bfloat16*)table,
                                                               (const __nv_bfloat16*)pos_table, out, D);
    else
        return mllm_fail(1, "embed: unknown dtype code %d", dtype);
    MLLM_CHECK_LAUNCH("embed");
    return 0;
}

// ids[t] < 0 stands for "the token that the last sampling launch wrote to row -ids[t]-1 of
// its output": the step that consumes a token can be queued before the host has read it.
__global__ void resolve_tokens_kernel(int* __restrict__ ids, int T, const int* __restrict__ sampled, int rows) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int v = ids[t];
    if (v < 0) {
        const int r = -v - 1;
        ids[t] = r < rows ? sampled[r] : 0;
    }
}

MLLM_EXPORT int mllm_resolve_tokens(int* ids, int T, const int* sampled, int rows, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rows <= 0) return mllm_fail(1, "resolve_tokens: no sampled rows to read from");
    resolve_tokens_kernel<<<(T + 255) / 256, 256, 0, stream>>>(ids, T, sampled, rows);
    MLLM_CHECK_LAUNCH("resolve_tokens");
    return 0;
}
