// Shared helpers of the sm_100a kernels: error reporting to the host, dtype
// codes, loads that widen to 32-bit, block reductions with a fixed order.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#define MLLM_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes used across the C interface
enum { MLLM_F32 = 0, MLLM_BF16 = 1 };
// epilogue activation codes
enum { MLLM_ACT_NONE = 0, MLLM_ACT_GELU_TANH = 1, MLLM_ACT_GELU_ERF = 2 };

// Records a message for mllm_last_error() and returns the code.
int mllm_fail(int code, const char* fmt, ...);

#define MLLM_CHECK_LAUNCH(name)                                                   \
    do {                                                                          \
        cudaError_t e__ = cudaGetLastError();                                     \
        if (e__ != cudaSuccess)                                                   \
            return mllm_fail(2, "%s: launch failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

#define MLLM_CUDA(call)                                                           \
    do {                                                                          \
        cudaError_t e__ = (call);                                                 \
        if (e__ != cudaSuccess)                                                   \
            return mllm_fail(3, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

// Programmatic dependent launch: a kernel launched with the attribute may start while the
// kernel before it on the stream is still running.  pdl_wait() returns once that kernel has
// completed and its writes are visible; until then only data that no kernel of the step
// writes (weights) may be touched.  pdl_launch() lets the kernel after this one start its
// own prologue.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1: launches that allow it carry the programmatic-serialization attribute (mllm_set_pdl).
extern int g_mllm_pdl;

template <typename... KArgs, typename... Args>
inline cudaError_t mllm_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && g_mllm_pdl) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; every thread gets the result.  `scratch` holds 33 floats.
// The order of additions depends only on blockDim, never on the data or the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read by an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// tanh-GELU as the reference writes it (src/kernels/gemm.cu:17-20) and the erf form.
__device__ __forceinline__ float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608f * (v + 0.044715f * v * v * v)));
}
__device__ __forceinline__ float gelu_erf_f(float v) {
    return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
}
// The tanh form written with one exponential, for epilogues whose result is rounded to
// bfloat16: 0.5*v*(1+tanh(u)) = v / (1 + exp(-2u)).  __expf and the reciprocal are good to
// about 1e-6 relative, far below the bfloat16 rounding that follows.
__device__ __forceinline__ float gelu_tanh_fast(float v) {
    const float u = 0.7978845608f * (v + 0.044715f * v * v * v);
    return __fdividef(v, 1.0f + __expf(-2.0f * u));
}
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == MLLM_ACT_GELU_TANH) return gelu_tanh_f(v);
    if (act == MLLM_ACT_GELU_ERF) return gelu_erf_f(v);
    return v;
}
