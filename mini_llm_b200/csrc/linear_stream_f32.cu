// out = act(LN?(x)[M,K] . W[N,K]^T + bias) (+ out) for up to 64 rows in true 32-bit (fmaf on CUDA cores,
// no tensor core, no reduced-precision mode): the products of decode steps on the float32 path, where
// the time goes into streaming the 32-bit weights from HBM once and into the dependent round trips
// between the kernels of a step.
//
// A CTA of 8 warps owns 8 weight rows (and, when the matrix has too few rows to fill the GPU, a slice of
// K: the CTAs of a thread-block cluster share a tile's K and meet in distributed shared memory).  Thread 0
// brings the CTA's weights into shared memory with bulk copies (cp.async.bulk onto an mbarrier, one copy
// per row) BEFORE the kernel waits for its predecessor: weights depend on no kernel of the step, so they
// stream from HBM while the previous kernel still runs, and no register is held for them.  After the wait
// every warp takes whole tokens (warp w the tokens w, w+8, ...; up to 8 per warp), its lanes split K in
// float4 steps of 128, x comes straight from L2 and the weights from shared memory, conflict-free.
// A token's sum runs over k in an order that depends on K and on the K slices only (lane partial sums
// in k order, a butterfly over the lanes, slices in rank order): never on M, so a token's result does
// not change with the batch.
//
// Fused on the input (up to 16 rows, no K slices): LayerNorm of the 32-bit residual rows, optionally
// gathered by `rows`; the warp that owns a token holds its row in registers, computes mean and variance
// in two passes as the separate norm kernel does, and multiplies the normalised values.  Fused on the
// output: bias, activation, the residual sum, and for a Q|K|V projection the write of the key and value
// columns to their page slots.
//
// The reference's small-M kernel is a 1x32 SIMT tile chosen for M < 4 and the four GPT-2-small shapes
// (src/kernels/decode_gemm.cu:42-134, 171-210); its norm, cache write and products are separate
// launches (src/model/gpt2_model.cu:487-541).
#include "tcgen05.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {

constexpr int WARPS = 8;
constexpr int R = 8;                    // weight rows per CTA
constexpr int MAX_M = 64;
constexpr int MAX_SLICES = 4;

__device__ int g_stream_error = 0;      // 1: the weights of a CTA never arrived (bounded wait ran out)

struct LnArgs {
    const float* x;          // [*, K] 32-bit residual rows, row stride ldx
    const int* rows;         // optional gather
    const float* gamma;
    const float* beta;
    float eps;
};
struct KvArgs {
    float* k_pages;          // [page][kv_head][offset][head_dim]
    float* v_pages;
    const int* slots;        // slot = page * page_size + offset, per token
    int q_size, kv_heads, head_dim, page_size;
};

__device__ __forceinline__ float dot4(const float4& w, const float4& x, float acc) {
    acc = fmaf(w.x, x.x, acc);
    acc = fmaf(w.y, x.y, acc);
    acc = fmaf(w.z, x.z, acc);
    return fmaf(w.w, x.w, acc);
}

// TPW: tokens per warp.  KC: with LN, float4 steps of a row that a lane keeps (rows up to KC*128 wide); 0 = no norm.
template <int TPW, int KC, bool KVW>
__global__ void __launch_bounds__(WARPS * 32)
linear_stream_f32_kernel(const float* x, long long ldx, const float* __restrict__ W, const float* __restrict__ bias,
                         float* out, long long ldo, int M, int N, int K, int Ks, int S, int act, int accumulate,
                         LnArgs ln, KvArgs kv) {
    constexpr bool LN = KC > 0;
    extern __shared__ __align__(16) float smem[];
    __shared__ __align__(8) uint64_t s_bar;
    float* ws = smem;                                   // [R][Ks] this CTA's weights
    float* part = smem + (size_t)R * Ks;                // S > 1, rank 0: [S][MAX_M][R] partial sums; LN: gamma | beta
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = S > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int n0 = (blockIdx.x / S) * R;
    const int rows = min(R, N - n0);
    const int k_lo = rank * Ks, k_hi = min(K, k_lo + Ks);
    const int kn = max(0, k_hi - k_lo);                  // a multiple of 4, as K and Ks are

    if (threadIdx.x == 0) {
        tc::mbar_init(&s_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::mbar_expect_tx(&s_bar, (uint32_t)(rows * kn) * 4u);
        if (kn > 0)
            for (int r = 0; r < rows; ++r)
                tc::bulk_load(ws + (size_t)r * Ks, W + (size_t)(n0 + r) * K + k_lo, (uint32_t)kn * 4u, &s_bar);
    }
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "I run": completes once all do
    if constexpr (LN) {
        // gamma and beta are weights as well: into shared memory before the wait
        for (int k = threadIdx.x * 4; k < K; k += WARPS * 32 * 4) {
            *reinterpret_cast<float4*>(part + k) = __ldg(reinterpret_cast<const float4*>(ln.gamma + k));
            *reinterpret_cast<float4*>(part + K + k) = __ldg(reinterpret_cast<const float4*>(ln.beta + k));
        }
    }
    pdl_wait();                 // everything below reads what earlier kernels of the step wrote
    pdl_launch();
    __syncthreads();            // the barrier is initialised, gamma and beta are in place

    // the residual values that this lane's outputs are added to, fetched early: lane r finishes row n0 + r
    const int e_n = n0 + lane;
    const bool e_ok = lane < rows && rank == 0;
    float e_old[TPW];
    int e_slot[TPW];
#pragma unroll
    for (int j = 0; j < TPW; ++j) {
        const int m = warp + j * WARPS;
        e_old[j] = 0.f;
        e_slot[j] = 0;
        if (e_ok && m < M) {
            if (KVW && e_n >= kv.q_size) e_slot[j] = __ldcg(kv.slots + m);
            else if (accumulate) e_old[j] = __ldcg(out + (size_t)m * ldo + e_n);
        }
    }

    float acc[R][TPW];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < TPW; ++j) acc[r][j] = 0.f;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    bool arrived = true;

    if constexpr (LN) {
        // the rows of this warp's tokens, whole, in registers; mean and variance in two passes
        float4 xr[TPW][KC];
#pragma unroll
        for (int j = 0; j < TPW; ++j) {
            const int m = warp + j * WARPS;
            const float* row = ln.x + (size_t)((m < M && ln.rows) ? __ldcg(ln.rows + m) : (m < M ? m : 0)) * ldx;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const int k = c * 128 + lane * 4;
                xr[j][c] = (m < M && k < K) ? __ldcg(reinterpret_cast<const float4*>(row + k)) : zero4;
            }
        }
#pragma unroll
        for (int j = 0; j < TPW; ++j) {
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < KC; ++c) s += (xr[j][c].x + xr[j][c].y) + (xr[j][c].z + xr[j][c].w);
            const float mean = warp_sum(s) / (float)K;
            float v = 0.f;
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                if (c * 128 + lane * 4 < K) {
                    const float a = xr[j][c].x - mean, b = xr[j][c].y - mean, cc = xr[j][c].z - mean, d = xr[j][c].w - mean;
                    v += (a * a + b * b) + (cc * cc + d * d);
                }
            }
            const float rstd = rsqrtf(warp_sum(v) / (float)K + ln.eps);
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const int k = c * 128 + lane * 4;
                if (k < K) {
                    const float4 g = *reinterpret_cast<const float4*>(part + k);
                    const float4 b = *reinterpret_cast<const float4*>(part + K + k);
                    xr[j][c].x = (xr[j][c].x - mean) * rstd * g.x + b.x;
                    xr[j][c].y = (xr[j][c].y - mean) * rstd * g.y + b.y;
                    xr[j][c].z = (xr[j][c].z - mean) * rstd * g.z + b.z;
                    xr[j][c].w = (xr[j][c].w - mean) * rstd * g.w + b.w;
                }
            }
        }
        arrived = tc::mbar_wait(&s_bar, 0);
        if (arrived) {
#pragma unroll
            for (int c = 0; c < KC; ++c) {
                const int k = c * 128 + lane * 4;
                if (k < kn) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float4 w = r < rows ? *reinterpret_cast<const float4*>(ws + (size_t)r * Ks + k) : zero4;
#pragma unroll
                        for (int j = 0; j < TPW; ++j) acc[r][j] = dot4(w, xr[j][c], acc[r][j]);
                    }
                }
            }
        }
    } else {
        // x in steps of 128 floats per warp, the next step's values on their way while this one is multiplied
        const int nsteps = (kn + 127) / 128;
        float4 xc[TPW], xn[TPW];
        auto load_x = [&](int c, float4 (&dst)[TPW]) {
            const int k = c * 128 + lane * 4;
#pragma unroll
            for (int j = 0; j < TPW; ++j) {
                const int m = warp + j * WARPS;
                dst[j] = (m < M && k < kn) ? __ldcg(reinterpret_cast<const float4*>(x + (size_t)m * ldx + k_lo + k)) : zero4;
            }
        };
        if (nsteps > 0) load_x(0, xc);
        arrived = tc::mbar_wait(&s_bar, 0);
        if (arrived) {
            for (int c = 0; c < nsteps; ++c) {
                if (c + 1 < nsteps) load_x(c + 1, xn);
                const int k = c * 128 + lane * 4;
                if (k < kn) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float4 w = r < rows ? *reinterpret_cast<const float4*>(ws + (size_t)r * Ks + k) : zero4;
#pragma unroll
                        for (int j = 0; j < TPW; ++j) acc[r][j] = dot4(w, xc[j], acc[r][j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < TPW; ++j) xc[j] = xn[j];
            }
        }
    }
    if (!arrived && lane == 0) {          // gave up: tell the host; the sums stay zero, the step's results are not used
        atomicCAS(&g_stream_error, 0, 1);
        tc::report_to_host(401);
    }

    // lanes' partial sums meet; afterwards lane r holds row r's sum of every token of the warp
    float v[TPW];
#pragma unroll
    for (int j = 0; j < TPW; ++j) v[j] = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < TPW; ++j) {
            const float s = warp_sum(acc[r][j]);
            if (lane == r) v[j] = s;
        }

    if (S > 1) {
        // every rank leaves its partial sums in rank 0's shared memory; rank 0 adds them in rank order
        cg::cluster_group cluster = cg::this_cluster();
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");       // rank 0 runs: its memory may be written
        float* dst = cluster.map_shared_rank(part, 0) + (size_t)rank * MAX_M * R;
        if (lane < R) {
#pragma unroll
            for (int j = 0; j < TPW; ++j) {
                const int m = warp + j * WARPS;
                if (m < M) dst[m * R + lane] = v[j];
            }
        }
        cluster.sync();                                                            // all partial sums are in place
        if (rank != 0) return;
        if (lane < R) {
#pragma unroll
            for (int j = 0; j < TPW; ++j) {
                const int m = warp + j * WARPS;
                if (m < M) {
                    float s = part[m * R + lane];
                    for (int q = 1; q < S; ++q) s += part[(size_t)q * MAX_M * R + m * R + lane];
                    v[j] = s;
                }
            }
        }
    }

    if (e_ok) {
        const float b = bias ? __ldg(bias + e_n) : 0.f;
#pragma unroll
        for (int j = 0; j < TPW; ++j) {
            const int m = warp + j * WARPS;
            if (m >= M) continue;
            float val = apply_act(v[j] + b, act);
            if (KVW && e_n >= kv.q_size) {
                const int kvw = kv.kv_heads * kv.head_dim;
                const int c = e_n - kv.q_size;
                float* pages = c < kvw ? kv.k_pages : kv.v_pages;
                const int cc = c < kvw ? c : c - kvw;
                const int head = cc / kv.head_dim, d = cc % kv.head_dim;
                const int page = e_slot[j] / kv.page_size, off = e_slot[j] % kv.page_size;
                pages[(((size_t)page * kv.kv_heads + head) * kv.page_size + off) * kv.head_dim + d] = val;
            } else {
                if (accumulate) val += e_old[j];
                out[(size_t)m * ldo + e_n] = val;
            }
        }
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

}  // namespace

// K slices that the CTAs of a cluster share, chosen from the matrix alone (never from M): a matrix with few
// rows gets slices until its CTAs fill the GPU twice, as long as a slice keeps at least 256 of K.
MLLM_EXPORT int mllm_linear_stream_f32_slices(int N, int K) {
    int S = 1;
    const int tiles = (N + R - 1) / R;
    while (S < MAX_SLICES && tiles * S < 2 * sm_count() && K / (2 * S) >= 256) S *= 2;
    return S;
}

MLLM_EXPORT int mllm_linear_stream_f32_bind_error(int* word) { return tc::bind_host_error(word); }

MLLM_EXPORT int mllm_linear_stream_f32_error(int* code) {
    int zero = 0;
    MLLM_CUDA(cudaMemcpyFromSymbol(code, g_stream_error, sizeof(int)));
    if (*code) MLLM_CUDA(cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int)));
    return 0;
}

// float32 x [M,K] (row stride ldx) or, when ln_x is given, LayerNorm(ln_x[ln_rows]) with gamma, beta, eps;
// W [N,K]; out [M,N] (row stride ldo).  With k_pages the columns from q_size on are keys, then values, and go
// to the page slots `slots[m]` instead of `out`.  Needs M <= 64 (16 with the norm), K a multiple of 4 (at most
// 2048 with the norm), 16-byte aligned x, W, gamma, beta and row strides that are multiples of 4.
MLLM_EXPORT int mllm_linear_stream_f32(const void* x, long long ldx, const void* W, const float* bias, void* out,
                                       long long ldo, int M, int N, int K, int act, int accumulate,
                                       const void* ln_x, const int* ln_rows, const float* ln_gamma,
                                       const float* ln_beta, float ln_eps, void* k_pages, void* v_pages,
                                       const int* slots, int q_size, int kv_heads, int head_dim, int page_size,
                                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    const bool norm = ln_x != nullptr;
    const bool kvw = k_pages != nullptr;
    if (M > MAX_M || (norm && M > 16)) return mllm_fail(1, "linear_stream_f32: M=%d exceeds %d", M, norm ? 16 : MAX_M);
    if (K <= 0 || K % 4 != 0 || ldx % 4 != 0 || (uintptr_t)(norm ? ln_x : x) % 16 != 0 || (uintptr_t)W % 16 != 0)
        return mllm_fail(1, "linear_stream_f32: K and the row stride must be multiples of 4, operands 16-byte aligned");
    if (norm && (K > 2048 || (uintptr_t)ln_gamma % 16 || (uintptr_t)ln_beta % 16 || !ln_gamma || !ln_beta))
        return mllm_fail(1, "linear_stream_f32: the fused norm takes rows up to 2048 wide and aligned gamma and beta");
    if (kvw && (!v_pages || !slots || kv_heads <= 0 || head_dim <= 0 || page_size <= 0 ||
                N != q_size + 2 * kv_heads * head_dim || accumulate))
        return mllm_fail(1, "linear_stream_f32: cache write arguments do not fit N=%d", N);
    int S = norm ? 1 : mllm_linear_stream_f32_slices(N, K);
    int Ks = ((K + S - 1) / S + 3) / 4 * 4;
    size_t smem = (size_t)R * Ks * 4 + (norm ? (size_t)2 * K * 4 : (S > 1 ? (size_t)S * MAX_M * R * 4 : 0));
    while (smem > 200 * 1024 && S < MAX_SLICES && !norm) {          // rows too long for shared memory: more slices
        S *= 2;
        Ks = ((K + S - 1) / S + 3) / 4 * 4;
        smem = (size_t)R * Ks * 4 + (size_t)S * MAX_M * R * 4;
    }
    if (smem > 200 * 1024) return mllm_fail(1, "linear_stream_f32: K=%d is too long for shared memory", K);
    const int tiles = (N + R - 1) / R;
    LnArgs ln = {(const float*)ln_x, ln_rows, ln_gamma, ln_beta, ln_eps};
    KvArgs kv = {(float*)k_pages, (float*)v_pages, slots, q_size, kv_heads, head_dim, page_size};
    const int tpw = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    const int kc = !norm ? 0 : K <= 1024 ? 8 : 16;
    using Kern = void (*)(const float*, long long, const float*, const float*, float*, long long, int, int, int, int,
                          int, int, int, LnArgs, KvArgs);
    Kern kern = nullptr;
#define PICK(T, C)                                                                              \
    if (tpw == T && kc == C)                                                                    \
        kern = kvw ? (Kern)linear_stream_f32_kernel<T, C, true> : (Kern)linear_stream_f32_kernel<T, C, false>;
    PICK(1, 0) PICK(2, 0) PICK(4, 0) PICK(8, 0) PICK(1, 8) PICK(2, 8) PICK(1, 16) PICK(2, 16)
#undef PICK
    if (!kern) return mllm_fail(1, "linear_stream_f32: no kernel for M=%d with%s norm", M, norm ? "" : "out");
    if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * S);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (S > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = S;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (g_mllm_pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    MLLM_CUDA(cudaLaunchKernelEx(&cfg, kern, (const float*)x, ldx, (const float*)W, bias, (float*)out, ldo, M, N, K, Ks, S,
                                 act, accumulate, ln, kv));
    return 0;
}
