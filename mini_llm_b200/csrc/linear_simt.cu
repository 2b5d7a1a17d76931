// out = act(A[M,K] . W[N,K]^T + bias[N]) (+ out): the plain matrix product of the
// engine, on CUDA cores with 32-bit FMA accumulation.
//
// It is the whole product path of the true 32-bit mode (float operands: no tensor
// core, no reduced-precision matrix mode) and the plain twin that the tensor-core
// kernels are tested against (bfloat16 operands widened to 32-bit).  Both operands
// are read along K, the layout every weight is brought to at load, so the tied head
// uses the embedding table as it is; the reference multiplies row-major [K,N]
// weights with its own SGEMM tiles (src/kernels/gemm.cu:238-392) and fuses the same
// epilogues: bias (src/kernels/linear.cu:8-26), bias+GELU (:48-66), bias+residual as
// beta=1 (:28-46).
//
// The sum over K of one output element always runs in the same order: K tiles in
// sequence and, for 32-bit products of many rows with a narrow result, a fixed number
// of K slices (chosen from N and K alone) whose partial sums a second kernel adds in
// slice order.  So a row's result does not depend on M or on the rows beside it.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int THREADS = (BM / TM) * (BN / TN);   // 256
constexpr int PAD = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* base, long long ld, int row, int nrows, int k, int K,
                                      bool vec, float (&v)[4]) {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (row >= nrows) return;
    const T* p = base + (size_t)row * ld + k;
    if (vec && k + 3 < K) {
        if constexpr (sizeof(T) == 4) {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            const uint2 u = *reinterpret_cast<const uint2*>(p);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
            v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (k + i < K) v[i] = to_f32(p[i]);
    }
}

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(THREADS)
linear_simt_kernel(const TA* A, long long lda, const TW* __restrict__ W, const float* __restrict__ bias,
                   TO* out, long long ldo, int M, int N, int K, int act, int accumulate, int vecA, int vecW) {
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lrow = tid / 4, lk = (tid % 4) * 4;      // 64 rows x 16 k: 4 consecutive k per thread
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4], w[4];
        load4<TA>(A, lda, m0 + lrow, M, k0 + lk, K, vecA != 0, a);
        load4<TW>(W, (long long)K, n0 + lrow, N, k0 + lk, K, vecW != 0, w);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lrow] = a[i];
            Ws[lk + i][lrow] = w[i];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * TM]);
            const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * TN]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = apply_act(v, act);
            TO* o = out + (size_t)m * ldo + n;
            if (accumulate) v += to_f32(*o);
            *o = from_f32<TO>(v);
        }
    }
}

// The same product with 128 x 128 tiles and 8 x 8 outputs per thread (as 2 x 2 blocks of 4 x 4),
// for many rows: four times the arithmetic per byte read from shared memory, and the next K tile
// is fetched into registers while the current one is multiplied.  Same order of the sum over K.
constexpr int LBM = 128, LBN = 128, LBK = 16, LTHREADS = 256;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(LTHREADS)        // one CTA per SM as compiled (129 registers); forcing two was slower (measured)
linear_simt_large_kernel(const TA* A, long long lda, const TW* __restrict__ W,
                         const float* __restrict__ bias, TO* out, long long ldo, int M, int N, int K_all, int act,
                         int accumulate, int vecA, int vecW, int splits, float* ws) {
    __shared__ float As[2][LBK][LBM + 4];
    __shared__ float Ws[2][LBK][LBN + 4];
    pdl_wait();
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * LBM, n0 = blockIdx.x * LBN;
    // K slice of this CTA (blockIdx.z): whole K tiles, so that slices start on aligned addresses
    const int kslice = ((K_all + splits - 1) / splits + LBK - 1) / LBK * LBK;
    const int k_begin = blockIdx.z * kslice;
    const int K = min(K_all, k_begin + kslice);
    const int lrow = tid / 2, lk = (tid % 2) * 8;       // 128 rows x 16 k: 8 consecutive k per thread
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    float a0[4], a1[4], w0[4], w1[4];
    auto fetch = [&](int k0) {
        load4<TA>(A, lda, m0 + lrow, M, k0 + lk, K, vecA != 0, a0);
        load4<TA>(A, lda, m0 + lrow, M, k0 + lk + 4, K, vecA != 0, a1);
        load4<TW>(W, (long long)K_all, n0 + lrow, N, k0 + lk, K, vecW != 0, w0);
        load4<TW>(W, (long long)K_all, n0 + lrow, N, k0 + lk + 4, K, vecW != 0, w1);
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[buf][lk + i][lrow] = a0[i];
            As[buf][lk + 4 + i][lrow] = a1[i];
            Ws[buf][lk + i][lrow] = w0[i];
            Ws[buf][lk + 4 + i][lrow] = w1[i];
        }
    };
    fetch(k_begin);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = k_begin; k0 < K; k0 += LBK) {
        const bool more = k0 + LBK < K;
        if (more) fetch(k0 + LBK);
#pragma unroll
        for (int k = 0; k < LBK; ++k) {
            const float4 al = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
            const float4 ah = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
            const float4 wl = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
            const float4 wh = *reinterpret_cast<const float4*>(&Ws[buf][k][64 + tx * 4]);
            const float ar[8] = {al.x, al.y, al.z, al.w, ah.x, ah.y, ah.z, ah.w};
            const float wr[8] = {wl.x, wl.y, wl.z, wl.w, wh.x, wh.y, wh.z, wh.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
            if (n >= N) continue;
            float v = acc[i][j];
            if (splits > 1) {                     // a slice's partial sum: the finishing kernel adds the slices in order
                ws[((size_t)blockIdx.z * M + m) * N + n] = v;
                continue;
            }
            if (bias) v += bias[n];
            v = apply_act(v, act);
            TO* o = out + (size_t)m * ldo + n;
            if (accumulate) v += to_f32(*o);
            *o = from_f32<TO>(v);
        }
    }
}

// out = act(ws[0] + ws[1] + ... + bias) (+ out): the K slices of the kernel above, added in slice order.
template <typename TO>
__global__ void __launch_bounds__(256)
linear_simt_finish_kernel(const float* __restrict__ ws, int splits, const float* __restrict__ bias, TO* out,
                          long long ldo, int M, int N, int act, int accumulate) {
    const size_t total = (size_t)M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / N), n = (int)(i % N);
        float v = __ldcg(ws + i);
        for (int z = 1; z < splits; ++z) v += __ldcg(ws + (size_t)z * total + i);
        if (bias) v += bias[n];
        v = apply_act(v, act);
        TO* o = out + (size_t)m * ldo + n;
        if (accumulate) v += to_f32(*o);
        *o = from_f32<TO>(v);
    }
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 148;
    }
    return n;
}

// K slices of the 32-bit product with many rows, from N and K alone: a result with few 128-column tiles gets slices
// until its CTAs at 2,048 rows (16 row tiles) come near one wave of two CTAs per SM; a slice keeps at least 256 of K.
int simt_splits(int N, int K) {
    const int cols = (N + LBN - 1) / LBN;
    int s = (2 * sm_count() / 16 + cols / 2) / cols;
    if (s > 4) s = 4;
    while (s > 1 && K / s < 256) --s;
    return s < 1 ? 1 : s;
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, long long lda, const void* W, const float* bias, void* out, long long ldo, int M, int N,
           int K, int act, int accumulate, float* ws, long long ws_floats, cudaStream_t stream) {
    const bool vecA = ((uintptr_t)A % (4 * sizeof(TA)) == 0) && (lda % 4 == 0);
    const bool vecW = ((uintptr_t)W % (4 * sizeof(TW)) == 0) && (K % 4 == 0);
    if (M > 128 && N >= 128 && (M + LBM - 1) / LBM <= 65535) {
        int splits = 1;
        if (sizeof(TA) == 4 && sizeof(TO) == 4 && ws) {
            splits = simt_splits(N, K);
            if ((long long)splits * M * N > ws_floats) splits = 1;        // no room for the partial sums (never, with ops.py)
        }
        dim3 lgrid((N + LBN - 1) / LBN, (M + LBM - 1) / LBM, splits);
        linear_simt_large_kernel<TA, TW, TO><<<lgrid, LTHREADS, 0, stream>>>(
            (const TA*)A, lda, (const TW*)W, bias, (TO*)out, ldo, M, N, K, act, accumulate, vecA, vecW, splits, ws);
        MLLM_CHECK_LAUNCH("linear_simt_large");
        if (splits > 1) {
            const size_t total = (size_t)M * N;
            const int blocks = (int)((total + 256 * 4 - 1) / (256 * 4));
            linear_simt_finish_kernel<TO><<<blocks, 256, 0, stream>>>(ws, splits, bias, (TO*)out, ldo, M, N, act, accumulate);
            MLLM_CHECK_LAUNCH("linear_simt_finish");
        }
        return 0;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    linear_simt_kernel<TA, TW, TO><<<grid, THREADS, 0, stream>>>(
        (const TA*)A, lda, (const TW*)W, bias, (TO*)out, ldo, M, N, K, act, accumulate, vecA, vecW);
    MLLM_CHECK_LAUNCH("linear_simt");
    return 0;
}

}  // namespace

// K slices that mllm_linear_simt uses for float32 operands and M > 128 rows (1: none).
MLLM_EXPORT int mllm_linear_simt_splits(int N, int K) { return simt_splits(N, K); }

// in_dtype: dtype of A and W; out_dtype: dtype of out.  ws (ws_floats floats, may be null): room for the partial
// sums of the K slices, mllm_linear_simt_splits(N, K) * M * N floats when that is more than one slice.
MLLM_EXPORT int mllm_linear_simt(const void* A, long long lda, const void* W, const float* bias, void* out,
                                 long long ldo, int M, int N, int K, int act, int accumulate, int in_dtype,
                                 int out_dtype, float* ws, long long ws_floats, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return mllm_fail(1, "linear: K=%d", K);
    if ((M + BM - 1) / BM > 65535) return mllm_fail(1, "linear: M=%d exceeds the grid limit of this kernel", M);
    using bf = __nv_bfloat16;
    if (in_dtype == MLLM_F32 && out_dtype == MLLM_F32)
        return launch<float, float, float>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, ws, ws_floats, stream);
    if (in_dtype == MLLM_BF16 && out_dtype == MLLM_BF16)
        return launch<bf, bf, bf>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, nullptr, 0, stream);
    if (in_dtype == MLLM_BF16 && out_dtype == MLLM_F32)
        return launch<bf, bf, float>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, nullptr, 0, stream);
    return mllm_fail(1, "linear: unsupported dtype pair in=%d out=%d", in_dtype, out_dtype);
}
