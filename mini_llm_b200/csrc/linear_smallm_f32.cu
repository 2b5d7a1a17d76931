// out = act(x[M,K] . W[N,K]^T + bias) (+ out) for few rows (M <= 16) in true 32-bit: the
// product of decode steps on the float32 path, where the time goes into streaming the
// 32-bit weights from HBM once.
//
// One warp per weight row: a lane reads 16 bytes of the row at k = 4*lane, 4*lane + 128, ...
// (512 contiguous bytes per warp and step, several steps in flight) and the matching values
// of every token's row of x (staged in shared memory once per CTA when they fit), multiplies with fmaf into one accumulator per
// token, and the warp adds its lanes' sums with shuffles.  The order of the additions
// depends on K only, so a token's result does not change with the batch.  No tensor core,
// no reduced-precision mode.  The reference's small-M kernel is a 1x32 SIMT tile
// (src/kernels/decode_gemm.cu:42-134).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

template <int MT>     // tokens held in registers: 4, 8 or 16
__global__ void __launch_bounds__(WARPS * 32)
linear_smallm_f32_kernel(const float* x, long long ldx, const float* __restrict__ W,
                         const float* __restrict__ bias, float* out, long long ldo, int M, int N, int K, int act,
                         int accumulate, int staged) {
    extern __shared__ __align__(16) float xs[];      // the M rows of x, when they fit (staged != 0)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * WARPS + warp;
    const bool active = n < N;                       // a warp beyond the matrix still helps staging x and meets the barrier
    const float* wr = W + (size_t)(active ? n : 0) * K;
    constexpr int U = 4;
    float4 w[U];
    auto load_w = [&](int k0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 128 + lane * 4;
            w[u] = (k < K && active) ? __ldcs(reinterpret_cast<const float4*>(wr + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    load_w(0);                   // weights do not depend on earlier kernels of the step
    pdl_wait();
    pdl_launch();
    if (staged) {
        // every warp of the CTA multiplies with the same rows of x: they come from L2 once, into shared memory
        for (int i = threadIdx.x * 4; i < M * K; i += WARPS * 32 * 4) {
            const int m = i / K, k = i % K;
            *reinterpret_cast<float4*>(xs + i) = __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * ldx + k));
        }
        __syncthreads();
    }
    if (!active) return;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    for (int k0 = 0; k0 < K; k0 += U * 128) {
        float4 cur[U];
#pragma unroll
        for (int u = 0; u < U; ++u) cur[u] = w[u];
        if (k0 + U * 128 < K) load_w(k0 + U * 128);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 128 + lane * 4;
            if (k >= K) continue;                    // K is a multiple of 4: a lane's 4 values are in or out together
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < M) {
                    const float4 xv = staged ? *reinterpret_cast<const float4*>(xs + (size_t)m * K + k)
                                             : __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * ldx + k));
                    acc[m] = fmaf(cur[u].x, xv.x, acc[m]);
                    acc[m] = fmaf(cur[u].y, xv.y, acc[m]);
                    acc[m] = fmaf(cur[u].z, xv.z, acc[m]);
                    acc[m] = fmaf(cur[u].w, xv.w, acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
    // lane m finishes token m
    float v = 0.f;
#pragma unroll
    for (int m = 0; m < MT; ++m)
        if (lane == m) v = acc[m];
    if (lane < M && lane < MT) {
        if (bias) v += bias[n];
        v = apply_act(v, act);
        float* o = out + (size_t)lane * ldo + n;
        if (accumulate) v += *o;
        *o = v;
    }
}

}  // namespace

// float32 x [M,K] (row stride ldx), W [N,K], out [M,N] (row stride ldo).  Needs M <= 16, K a
// multiple of 4, 16-byte aligned x and W and ldx a multiple of 4.
MLLM_EXPORT int mllm_linear_smallm_f32(const void* x, long long ldx, const void* W, const float* bias, void* out,
                                       long long ldo, int M, int N, int K, int act, int accumulate,
                                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16) return mllm_fail(1, "linear_smallm_f32: M=%d exceeds 16", M);
    if (K <= 0 || K % 4 != 0 || ldx % 4 != 0 || (uintptr_t)x % 16 != 0 || (uintptr_t)W % 16 != 0)
        return mllm_fail(1, "linear_smallm_f32: K and the row stride must be multiples of 4, operands 16-byte aligned");
    const int grid = (N + WARPS - 1) / WARPS;
    const size_t want = (size_t)M * K * sizeof(float);
    const int staged = want <= 96 * 1024;            // else the rows of x are read from L2 as they are needed
    const size_t smem = staged ? want : 0;
#define GO(MT)                                                                                                    \
    {                                                                                                             \
        auto kern = linear_smallm_f32_kernel<MT>;                                                                 \
        static size_t set = 0;                                                                                    \
        if (smem > 48 * 1024 && smem > set) {                                                                     \
            MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(96 * 1024))); \
            set = 96 * 1024;                                                                                      \
        }                                                                                                         \
        MLLM_CUDA(mllm_launch(kern, dim3(grid), dim3(WARPS * 32), smem, stream, true, (const float*)x, ldx,      \
                              (const float*)W, bias, (float*)out, ldo, M, N, K, act, accumulate, staged));        \
        return 0;                                                                                                 \
    }
    if (M <= 4) GO(4)
    if (M <= 8) GO(8)
    GO(16)
#undef GO
}
