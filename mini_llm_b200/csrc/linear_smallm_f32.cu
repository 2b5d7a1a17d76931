// out = act(x[M,K] . W[N,K]^T + bias) (+ out) for few rows (M <= 16) in true 32-bit: the
// product of decode steps on the float32 path, where the time goes into streaming the
// 32-bit weights from HBM once.
//
// One warp per weight row: a lane reads 16 bytes of the row at k = 4*lane, 4*lane + 128, ...
// (512 contiguous bytes per warp and step, several steps in flight) and the matching values
// of every token's row of x (from L1/L2), multiplies with fmaf into one accumulator per
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
                         int accumulate) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * WARPS + warp;
    if (n >= N) return;
    const float* wr = W + (size_t)n * K;
    constexpr int U = 4;
    float4 w[U];
    auto load_w = [&](int k0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * 128 + lane * 4;
            w[u] = k < K ? __ldcs(reinterpret_cast<const float4*>(wr + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    load_w(0);                   // weights do not depend on earlier kernels of the step
    pdl_wait();
    pdl_launch();
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
                    const float4 xv = __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * ldx + k));
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
#define GO(MT)                                                                                                    \
    MLLM_CUDA(mllm_launch(linear_smallm_f32_kernel<MT>, dim3(grid), dim3(WARPS * 32), 0, stream, true, (const float*)x, \
                          ldx, (const float*)W, bias, (float*)out, ldo, M, N, K, act, accumulate));               \
    return 0
    if (M <= 4) { GO(4); }
    if (M <= 8) { GO(8); }
    GO(16);
#undef GO
}
