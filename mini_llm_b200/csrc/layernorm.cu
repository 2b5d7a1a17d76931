// LayerNorm of 32-bit rows, optionally of gathered rows (the rows whose logits
// are wanted), written as 32-bit or bfloat16.
// mean; biased variance of the centred values; (x-mean)*rsqrt(var+eps)*gamma+beta,
// as src/kernels/layernorm.cu:32-49 of the reference, for any width (that kernel is
// fixed to 768 columns, :12).  One block per row; the row is re-read from L1/L2.
#include "common.cuh"

template <typename TOut>
__global__ void layernorm_kernel(const float* x, const int* __restrict__ rows,
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

// One warp per row, the row held in registers (up to 2048 columns): one read of the row, the
// centred second pass runs on registers, 16-byte loads and stores.  Same arithmetic order for
// a row whatever the number of rows.
template <typename TOut>
__global__ void __launch_bounds__(256)
layernorm_warp_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ gamma,
                      const float* __restrict__ beta, TOut* __restrict__ out, int R, int D, float eps) {
    constexpr int KEEP = 16;
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (r >= R) return;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float4 v[KEEP];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int k = lane * 4 + i * 128;
        v[i] = k < D ? *reinterpret_cast<const float4*>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = warp_sum(s) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        if (lane * 4 + i * 128 < D) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float inv = rsqrtf(warp_sum(q) / (float)D + eps);
    TOut* o = out + (size_t)r * D;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int k = lane * 4 + i * 128;
        if (k >= D) break;
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma + k));
        const float4 b = __ldg(reinterpret_cast<const float4*>(beta + k));
        const float y0 = (v[i].x - mean) * inv * g.x + b.x, y1 = (v[i].y - mean) * inv * g.y + b.y;
        const float y2 = (v[i].z - mean) * inv * g.z + b.z, y3 = (v[i].w - mean) * inv * g.w + b.w;
        if constexpr (sizeof(TOut) == 4) {
            *reinterpret_cast<float4*>(o + k) = make_float4(y0, y1, y2, y3);
        } else {
            uint2 pk;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
            h[0] = __floats2bfloat162_rn(y0, y1);
            h[1] = __floats2bfloat162_rn(y2, y3);
            *reinterpret_cast<uint2*>(o + k) = pk;
        }
    }
}

MLLM_EXPORT int mllm_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                               void* out, int R, int D, float eps, int out_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D <= 0) return mllm_fail(1, "layernorm: width %d", D);
    const bool fast = D % 4 == 0 && D <= 2048 && (uintptr_t)x % 16 == 0 && (uintptr_t)gamma % 16 == 0 &&
                      (uintptr_t)beta % 16 == 0 && (uintptr_t)out % 16 == 0;
    if (fast && (out_dtype == MLLM_F32 || out_dtype == MLLM_BF16)) {
        const int grid = (R + 7) / 8;
        if (out_dtype == MLLM_F32)
            MLLM_CUDA(mllm_launch(layernorm_warp_kernel<float>, dim3(grid), dim3(256), 0, stream, true, x, rows, gamma,
                                  beta, (float*)out, R, D, eps));
        else
            MLLM_CUDA(mllm_launch(layernorm_warp_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true, x, rows,
                                  gamma, beta, (__nv_bfloat16*)out, R, D, eps));
        return 0;
    }
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
