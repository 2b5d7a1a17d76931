// LayerNorm of 32-bit rows, optionally of gathered rows (the rows whose logits
// are wanted), written as 32-bit or bfloat16.
// mean; biased variance of the centred values; (x-mean)*rsqrt(var+eps)*gamma+beta,
// as src/kernels/layernorm.cu:32-49 of the reference, for any width (that kernel is
// fixed to 768 columns, :12).  One block per row; the row is re-read from L1/L2.
#include "common.cuh"

template <typename TOut>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 TOut* __restrict__ out, int D, float eps) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TOut* o = out + (size_t)r * D;
    float s = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) s += xr[d];
    const float mean = block_sum(s, scratch) / (float)D;
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float c = xr[d] - mean;
        q += c * c;
    }
    const float var = block_sum(q, scratch) / (float)D;
    const float inv = rsqrtf(var + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        o[d] = from_f32<TOut>((xr[d] - mean) * inv * gamma[d] + beta[d]);
}

MLLM_EXPORT int mllm_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                               void* out, int R, int D, float eps, int out_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D <= 0) return mllm_fail(1, "layernorm: width %d", D);
    int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : ((D + 31) / 32) * 32);
    if (out_dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(layernorm_kernel<float>, dim3(R), dim3(threads), 0, stream, true, x, rows, gamma, beta,
                              (float*)out, D, eps));
    else if (out_dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(layernorm_kernel<__nv_bfloat16>, dim3(R), dim3(threads), 0, stream, true, x, rows, gamma,
                              beta, (__nv_bfloat16*)out, D, eps));
    else
        return mllm_fail(1, "layernorm: unknown dtype code %d", out_dtype);
    MLLM_CHECK_LAUNCH("layernorm");
    return 0;
}
