// out = act(x[M,K] . W[N,K]^T + bias) (+ out) for few rows (M <= 64), bfloat16 operands:
// the product of the decode step, where every weight is read once and the time goes
// into streaming it from HBM.
//
// A CTA of 8 warps owns 16*RT weight rows.  The K dimension is cut into chunks of 32
// that the warps take in turn (warp w takes chunks w, w+8, ...), so at any moment the
// CTA reads 512 contiguous bytes of each of its rows.  A lane loads 16 bytes (8
// consecutive k) of two weight rows and of x straight from global memory into the
// fragments of two mma.sync.m16n8k16 (bf16 in, 32-bit accumulate): the k positions
// inside a chunk are permuted the same way for both operands, which a sum over k
// allows.  Tokens are the n dimension of the MMA (8 per tile, MT tiles).  Warp partial
// sums meet in shared memory and are added in warp order, then bias, activation and
// the residual sum (32-bit) are applied.  Nothing depends on M except which columns
// exist, so a token's result does not change with the batch.
//
// The reference's counterpart is decode_small_m_gemm_kernel, a 1x32 SIMT tile chosen
// for M < 4 and the four GPT-2-small shapes (src/kernels/decode_gemm.cu:42-134, 171-210).
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg16_cached(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int RT, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
linear_smallm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ W,
                     const float* __restrict__ bias, TO* out, long long ldo, int M, int N, int K, int act,
                     int accumulate) {
    extern __shared__ float red[];                 // [WARPS][16*RT][8*MT]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * (16 * RT);
    const int nchunks = (K + 31) / 32;
    constexpr int U = RT == 1 ? 4 : (RT == 2 ? 2 : 1);

    float acc[RT][MT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][m][i] = 0.f;

    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int c0 = warp; c0 < nchunks; c0 += WARPS * U) {
        uint4 wa[U][RT], wb[U][RT], xv[U][MT];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (c0 + u * WARPS) * 32 + 8 * t;
            const bool kok = k < K;                 // K is a multiple of 8: a lane's 8 values are in or out together
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                const int ra = n0 + r * 16 + g, rb = ra + 8;
                wa[u][r] = (kok && ra < N) ? ldg16(W + (size_t)ra * K + k) : zero;
                wb[u][r] = (kok && rb < N) ? ldg16(W + (size_t)rb * K + k) : zero;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int row = m * 8 + g;
                xv[u][m] = (kok && row < M) ? ldg16_cached(x + (size_t)row * ldx + k) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16(acc[r][m], wa[u][r].x, wb[u][r].x, wa[u][r].y, wb[u][r].y, xv[u][m].x, xv[u][m].y);
                    mma_bf16(acc[r][m], wa[u][r].z, wb[u][r].z, wa[u][r].w, wb[u][r].w, xv[u][m].z, xv[u][m].w);
                }
    }
    // partial sums of this warp -> shared memory
    constexpr int ROWS = 16 * RT, COLS = 8 * MT;
    float* mine = red + (size_t)warp * ROWS * COLS;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int row = r * 16 + g, col = m * 8 + 2 * t;
            mine[row * COLS + col] = acc[r][m][0];
            mine[row * COLS + col + 1] = acc[r][m][1];
            mine[(row + 8) * COLS + col] = acc[r][m][2];
            mine[(row + 8) * COLS + col + 1] = acc[r][m][3];
        }
    __syncthreads();
    // consecutive threads take consecutive weight rows (n) of one token, so stores run along n
    for (int i = threadIdx.x; i < ROWS * COLS; i += WARPS * 32) {
        const int row = i % ROWS, col = i / ROWS;
        const int n = n0 + row;
        if (n >= N || col >= M) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * ROWS * COLS + row * COLS + col];
        if (bias) v += bias[n];
        v = apply_act(v, act);
        TO* o = out + (size_t)col * ldo + n;
        if (accumulate) v += to_f32(*o);
        *o = from_f32<TO>(v);
    }
}

template <int MT, int RT, typename TO>
int launch(const void* x, long long ldx, const void* W, const float* bias, void* out, long long ldo, int M, int N,
           int K, int act, int accumulate, cudaStream_t stream) {
    const size_t smem = (size_t)WARPS * 16 * RT * 8 * MT * sizeof(float);
    auto kern = linear_smallm_kernel<MT, RT, TO>;
    if (smem > 48 * 1024) {
        static bool set = false;                   // per instantiation
        if (!set) {
            MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set = true;
        }
    }
    const int grid = (N + 16 * RT - 1) / (16 * RT);
    kern<<<grid, WARPS * 32, smem, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)W, bias, (TO*)out,
                                             ldo, M, N, K, act, accumulate);
    MLLM_CHECK_LAUNCH("linear_smallm");
    return 0;
}

template <int MT, typename TO>
int pick_rt(int rt, const void* x, long long ldx, const void* W, const float* bias, void* out, long long ldo, int M,
            int N, int K, int act, int accumulate, cudaStream_t stream) {
    if (rt == 4) return launch<MT, 4, TO>(x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    if (rt == 2) return launch<MT, 2, TO>(x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    return launch<MT, 1, TO>(x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
}

template <typename TO>
int pick_mt(int rt, const void* x, long long ldx, const void* W, const float* bias, void* out, long long ldo, int M,
            int N, int K, int act, int accumulate, cudaStream_t stream) {
    if (M <= 8) return pick_rt<1, TO>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    if (M <= 16) return pick_rt<2, TO>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    if (M <= 32) return pick_rt<4, TO>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    return pick_rt<8, TO>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
}

}  // namespace

// bfloat16 x and W; out bfloat16 or 32-bit.  Needs M <= 64, K a multiple of 8, and x
// and W 16-byte aligned with a row stride of x that is a multiple of 8.
MLLM_EXPORT int mllm_linear_smallm(const void* x, long long ldx, const void* W, const float* bias, void* out,
                                   long long ldo, int M, int N, int K, int act, int accumulate, int out_dtype,
                                   cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64) return mllm_fail(1, "linear_smallm: M=%d exceeds 64", M);
    if (K <= 0 || K % 8 != 0) return mllm_fail(1, "linear_smallm: K=%d is not a multiple of 8", K);
    if (ldx % 8 != 0 || (uintptr_t)x % 16 != 0 || (uintptr_t)W % 16 != 0)
        return mllm_fail(1, "linear_smallm: operands must be 16-byte aligned");
    // rows per CTA: enough CTAs to fill the 148 SMs when N allows it
    int rt = 1;
    if (N >= 16 * 4 * 296) rt = 4;
    else if (N >= 16 * 2 * 296) rt = 2;
    if (out_dtype == MLLM_BF16)
        return pick_mt<__nv_bfloat16>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    if (out_dtype == MLLM_F32)
        return pick_mt<float>(rt, x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    return mllm_fail(1, "linear_smallm: unknown dtype code %d", out_dtype);
}
