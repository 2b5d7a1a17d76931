// out = act(LN?(x)[M,K] . W[N,K]^T + bias) (+ out) for up to 64 rows in true 32-bit (fmaf on CUDA cores,
// no tensor core, no reduced-precision mode): the products of decode steps on the float32 path, where
// the time goes into streaming the 32-bit weights from HBM once and into the dependent round trips
// between the kernels of a step.
//
// A CTA of 8 warps owns tiles of 8 weight rows (and, when the matrix has too few rows to fill the GPU, a
// slice of K: the CTAs of a thread-block cluster share a tile's K and meet in distributed shared memory).
// Thread 0 brings the CTA's weights into shared memory with bulk copies (cp.async.bulk onto an mbarrier, one
// copy per row) BEFORE the kernel waits for its predecessor: weights depend on no kernel of the step, so
// they stream from HBM while the previous kernel still runs, and no register is held for them.
//
// Up to 16 rows of x (`few`): the threads split K.  Thread t takes the float4 positions t, t + 256, ... of
// the slice for all 8 weight rows and 8 tokens at a time, so every weight leaves shared memory once and
// every value of x leaves L2 once per CTA; the 64 sums of a thread meet first inside the warp (a butterfly
// that halves the values a lane holds at every step: 62 shuffles), then across the warps in shared memory
// in warp order, then across the slices in rank order.  17 to 64 rows (`many`): every warp takes whole
// tokens (warp w the tokens w, w + 8, ...), its lanes split K, and the weights are read from shared memory
// once per warp, which 8 tokens per warp amortise.
// Rows up to 2048 long (`tall`: the Q|K|V and up-projections, and the vocabulary) have a kernel whose CTAs stay on
// their SMs: x (normalised) in shared memory once per CTA, a warp's 4 or 2 weight rows in registers straight from
// HBM, no barrier in its loop.  It takes up to 16 rows of x, and for a matrix as tall as a vocabulary all that fit
// shared memory (64 at K = 768); where it was measured faster than the tile kernels is written beside its rule.
// A token's sum runs over k in an order that depends on N, K and on the slices only, never on M, so a
// token's result does not change with the batch (`few`, `many` and `tall` differ in rounding, as kernels do).
//
// Fused on the input (up to 16 rows, no K slices): LayerNorm of the 32-bit residual rows, optionally
// gathered by `rows`; a warp per token computes mean and variance in two passes from registers, as the
// separate norm kernel does, and the values are normalised as they are loaded.  Fused on the output:
// bias, activation, the residual sum, and for a Q|K|V projection the write of the key and value columns
// to their page slots.
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
constexpr int MAX_SLICES = 4;             // K slices of the kernel for up to 16 rows

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

// ---------------------------------------------------------------------------------------------------------
// Up to 16 rows: threads split K.

constexpr int FEW_M = 16;
constexpr int MAX_TILES = 4;            // tiles of R rows that one CTA may own

// One output of the epilogue: bias, activation, then either a cache slot or the (residual) output.
template <bool KVW>
__device__ __forceinline__ void finish_one(float v, int m, int n, float bias, float* out, long long ldo, int act,
                                           int accumulate, float old, int slot, const KvArgs& kv) {
    float val = apply_act(v + bias, act);
    if (KVW && n >= kv.q_size) {
        const int kvw = kv.kv_heads * kv.head_dim;
        const int c = n - kv.q_size;
        float* pages = c < kvw ? kv.k_pages : kv.v_pages;
        const int cc = c < kvw ? c : c - kvw;
        const int head = cc / kv.head_dim, d = cc % kv.head_dim;
        const int page = slot / kv.page_size, off = slot % kv.page_size;
        pages[(((size_t)page * kv.kv_heads + head) * kv.page_size + off) * kv.head_dim + d] = val;
    } else {
        if (accumulate) val += old;
        out[(size_t)m * ldo + n] = val;
    }
}

template <bool LN, bool KVW>
__global__ void __launch_bounds__(WARPS * 32, 2)
linear_stream_f32_few_kernel(const float* x, long long ldx, const float* __restrict__ W, const float* __restrict__ bias,
                             float* out, long long ldo, int M, int N, int K, int Ks, int S, int TILES, int act,
                             int accumulate, LnArgs ln, KvArgs kv) {
    extern __shared__ __align__(16) float smem[];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ float s_mean[FEW_M], s_rstd[FEW_M];
    float* ws = smem;                                       // [TILES * R][Ks] this CTA's weights
    float* red = ws + (size_t)TILES * R * Ks;               // [2][WARPS][64] the warps' sums, two buffers in turn
    float* part = red + 2 * WARPS * 64;                     // S > 1, rank 0: [S][2 groups][64] the slices' sums
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
    const int rank = S > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int n0 = (blockIdx.x / S) * TILES * R;
    const int rows_cta = max(0, min(TILES * R, N - n0));
    const int k_lo = rank * Ks, k_hi = min(K, k_lo + Ks);
    const int kn = max(0, k_hi - k_lo);                      // a multiple of 4, as K and Ks are
    const int npos = (kn / 4 + WARPS * 32 - 1) / (WARPS * 32);
    const int groups = (M + 7) / 8;

    if (t == 0) {
        tc::mbar_init(&s_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::mbar_expect_tx(&s_bar, (uint32_t)(rows_cta * kn) * 4u);
        if (kn > 0)
            for (int r = 0; r < rows_cta; ++r)
                tc::bulk_load(ws + (size_t)r * Ks, W + (size_t)(n0 + r) * K + k_lo, (uint32_t)kn * 4u, &s_bar);
    }
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "I run": completes once all do

    // Who finishes which output.  A pass over (token group g, tile tl) ends with 64 sums, token g * 8 + i / 8 and row
    // i % 8 of the tile.  The passes are numbered c = g * MAX_TILES + tl; the 64 threads with t / 64 == c % 4 finish
    // pass c, so a thread finishes at most two passes (c and c + 4) and keeps their bias, old value and cache slot
    // in registers, fetched long before they are needed.
    const int e_i = t & 63, e_m = e_i >> 3, e_r = e_i & 7, e_c = t >> 6;
    const int e_tl = e_c & (MAX_TILES - 1);                 // the same tile in both passes (c and c + 4 differ in g)
    const int e_n = n0 + e_tl * R + e_r;
    const bool e_col = e_tl < TILES && e_n < N && rank == 0;
    // gamma and beta at this thread's first position and the bias of its output column are weights too: before the wait
    float4 gam = make_float4(1.f, 1.f, 1.f, 1.f), bet = make_float4(0.f, 0.f, 0.f, 0.f);
    if constexpr (LN) {
        if (4 * t < kn) {
            gam = __ldg(reinterpret_cast<const float4*>(ln.gamma + 4 * t));
            bet = __ldg(reinterpret_cast<const float4*>(ln.beta + 4 * t));
        }
    }
    const float e_bias = (e_col && bias) ? __ldg(bias + e_n) : 0.f;
    pdl_wait();                 // everything below reads what earlier kernels of the step wrote
    pdl_launch();

    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* xbase = LN ? ln.x : x;
    auto row_of = [&](int m) -> const float* {
        return xbase + (size_t)((LN && ln.rows) ? __ldcg(ln.rows + m) : m) * ldx;
    };
    // every load of this thread that depends on the step goes out now, before anything waits for any of them
    float4 xv[8];
    auto load_x = [&](int g, int p) {
        const int k = 4 * (t + p * WARPS * 32);
#pragma unroll
        for (int m = 0; m < 8; ++m) {
            const int mm = g * 8 + m;
            xv[m] = (mm < M && k < kn) ? __ldcg(reinterpret_cast<const float4*>(row_of(mm) + k_lo + k)) : zero4;
        }
    };
    load_x(0, 0);
    float e_old[2] = {0.f, 0.f};
    int e_slot[2] = {0, 0};
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const int mm = g * 8 + e_m;
        if (e_col && mm < M) {
            if (KVW && e_n >= kv.q_size) e_slot[g] = __ldcg(kv.slots + mm);
            else if (accumulate) e_old[g] = __ldcg(out + (size_t)mm * ldo + e_n);
        }
    }

    if constexpr (LN) {
        // a warp per token: the row's first 1024 values in registers, what lies beyond (rows up to 2048 wide) is read a
        // second time for the variance; mean and variance in two passes, as the separate norm kernel computes them.
        // (Sums over the whole block of the values that the threads hold anyway were tried: two block-wide meetings
        // cost more than reading the rows a second time from L2.)
        for (int m = warp; m < M; m += WARPS) {
            const float* row = row_of(m);
            float4 rv[8];
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int k = c * 128 + lane * 4;
                rv[c] = k < K ? __ldcg(reinterpret_cast<const float4*>(row + k)) : zero4;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) sum += (rv[c].x + rv[c].y) + (rv[c].z + rv[c].w);
            for (int k = 1024 + lane * 4; k < K; k += 128) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(row + k));
                sum += (v.x + v.y) + (v.z + v.w);
            }
            const float mean = warp_sum(sum) / (float)K;
            float var = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (c * 128 + lane * 4 < K) {
                    const float a = rv[c].x - mean, b = rv[c].y - mean, cc = rv[c].z - mean, d = rv[c].w - mean;
                    var += (a * a + b * b) + (cc * cc + d * d);
                }
            }
            for (int k = 1024 + lane * 4; k < K; k += 128) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(row + k));
                const float a = v.x - mean, b = v.y - mean, cc = v.z - mean, d = v.w - mean;
                var += (a * a + b * b) + (cc * cc + d * d);
            }
            var = warp_sum(var) / (float)K;
            if (lane == 0) {
                s_mean[m] = mean;
                s_rstd[m] = rsqrtf(var + ln.eps);
            }
        }
    }
    __syncthreads();            // the barrier is initialised, the statistics are in place

    // the loaded values of x, normalised in place
    auto norm_x = [&](int g, int p) {
        if constexpr (LN) {
            const int k = 4 * (t + p * WARPS * 32);
            if (k >= kn) return;
            float4 gg = gam, bb = bet;
            if (p > 0) {
                gg = __ldg(reinterpret_cast<const float4*>(ln.gamma + k));
                bb = __ldg(reinterpret_cast<const float4*>(ln.beta + k));
            }
#pragma unroll
            for (int m = 0; m < 8; ++m) {
                const int mm = min(g * 8 + m, FEW_M - 1);
                const float mean = s_mean[mm], rstd = s_rstd[mm];
                xv[m].x = (xv[m].x - mean) * rstd * gg.x + bb.x;
                xv[m].y = (xv[m].y - mean) * rstd * gg.y + bb.y;
                xv[m].z = (xv[m].z - mean) * rstd * gg.z + bb.z;
                xv[m].w = (xv[m].w - mean) * rstd * gg.w + bb.w;
            }
        }
    };
    norm_x(0, 0);
    const bool arrived = tc::mbar_wait(&s_bar, 0);
    if (!arrived && t == 0) {             // gave up: tell the host; the results of the step are not used
        atomicCAS(&g_stream_error, 0, 1);
        tc::report_to_host(401);
    }
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // rank 0 runs: its memory may be written
    int buf = 0;
    for (int g = 0; g < groups; ++g) {
        for (int tl = 0; tl < TILES; ++tl) {
            float acc[64];                                   // [token][row]
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0.f;
            const int rows_tile = min(R, rows_cta - tl * R);
            for (int p = 0; p < npos; ++p) {
                if (!(g == 0 && tl == 0 && p == 0) && (npos > 1 || tl == 0)) {
                    load_x(g, p);
                    norm_x(g, p);
                }
                const int k = 4 * (t + p * WARPS * 32);
                if (k < kn && arrived) {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const float4 w = r < rows_tile ? *reinterpret_cast<const float4*>(ws + (size_t)(tl * R + r) * Ks + k) : zero4;
#pragma unroll
                        for (int m = 0; m < 8; ++m) acc[m * 8 + r] = dot4(w, xv[m], acc[m * 8 + r]);
                    }
                }
            }
            // inside the warp: at every step a lane hands half of its values to the lane `off` away and adds what
            // it gets to the half it keeps; afterwards lane l holds the warp's sums of the values 2l and 2l + 1
#pragma unroll
            for (int half = 32, off = 16; half >= 2; half >>= 1, off >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = upper ? acc[i] : acc[i + half];
                    const float keep = upper ? acc[i + half] : acc[i];
                    acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            float* rb = red + (size_t)buf * WARPS * 64;
            *reinterpret_cast<float2*>(rb + warp * 64 + 2 * lane) = make_float2(acc[0], acc[1]);
            __syncthreads();
            const int c = g * MAX_TILES + tl;
            if (e_c == (c & 3)) {                                             // the 64 threads that finish this pass
                float v = rb[e_i];
#pragma unroll
                for (int w = 1; w < WARPS; ++w) v += rb[w * 64 + e_i];         // warp order
                const int mm = g * 8 + e_m;
                if (S > 1) {
                    cluster.map_shared_rank(part, 0)[((size_t)rank * 2 + g) * 64 + e_i] = v;
                } else if (e_col && mm < M) {
                    finish_one<KVW>(v, mm, e_n, e_bias, out, ldo, act, accumulate, g ? e_old[1] : e_old[0],
                                    g ? e_slot[1] : e_slot[0], kv);
                }
            }
            buf ^= 1;
        }
    }
    if (S > 1) {
        cluster.sync();                                                        // every slice's sums are in place
        if (rank != 0) return;
        for (int g = 0; g < groups; ++g) {
            if (e_c == (g * MAX_TILES & 3)) {                                  // one tile per CTA when K is sliced
                float v = part[(size_t)g * 64 + e_i];
                for (int q = 1; q < S; ++q) v += part[((size_t)q * 2 + g) * 64 + e_i];   // rank order
                const int mm = g * 8 + e_m;
                if (e_col && mm < M)
                    finish_one<KVW>(v, mm, e_n, e_bias, out, ldo, act, accumulate, g ? e_old[1] : e_old[0],
                                    g ? e_slot[1] : e_slot[0], kv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// 17 to 64 rows: a CTA owns all tokens and a tile of RT = 4 * RJ weight rows (16, 24 or 32) over a slice of K; its
// 8 warps split the slice in chunks of 8 floats (warp w the chunks w, w + 8, ...), and inside a warp the lanes form
// 8 token groups x 4 row groups: lane (tg, rg) multiplies the tokens tg, tg + 8, ... with the rows rg, rg + 4, ...
// (8 x RJ sums per lane).  Per step of 4 floats of K a lane loads MI float4 of x straight from L2 (an address is
// shared by the 4 lanes of a token group: one request) and RJ float4 of the weights from shared memory (an address
// is shared by the 8 lanes of a row group: a broadcast), for 4 * MI * RJ fused multiply-adds.  The warps' tiles meet
// in shared memory in warp order, the slices' tiles in rank 0's shared memory in rank order.
constexpr int MANY_WS_PAD = 4;          // floats between weight rows in shared memory: row groups fall on different banks
constexpr int MANY_RED_PAD = 4;         // the same between token rows of the warps' partial tiles

template <int MI, int RJ, bool KVW>
__global__ void __launch_bounds__(WARPS * 32, 1)
linear_stream_f32_many_kernel(const float* x, long long ldx, const float* __restrict__ W, const float* __restrict__ bias,
                              float* out, long long ldo, int M, int N, int K, int Ks, int S, int act, int accumulate,
                              KvArgs kv) {
    constexpr int RT = 4 * RJ, MT = 8 * MI;
    extern __shared__ __align__(16) float smem[];
    __shared__ __align__(8) uint64_t s_bar;
    const int wstride = Ks + MANY_WS_PAD, rstride = RT + MANY_RED_PAD;
    float* ws = smem;                                       // [RT][Ks + pad] this CTA's weights
    float* red = ws + (size_t)RT * wstride;                 // [WARPS][MT][RT + pad] the warps' partial tiles
    float* part = red + (size_t)WARPS * MT * rstride;       // S > 1, rank 0: [S - 1][MT * RT] the other slices' tiles
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
    const int tg = lane >> 2, rg = lane & 3;
    const int rank = S > 1 ? (int)cg::this_cluster().block_rank() : 0;
    const int n0 = (blockIdx.x / S) * RT;
    const int rows = max(0, min(RT, N - n0));
    const int k_lo = rank * Ks, k_hi = min(K, k_lo + Ks);
    const int kn = max(0, k_hi - k_lo);                      // a multiple of 4, as K and Ks are

    if (t == 0) {
        tc::mbar_init(&s_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::mbar_expect_tx(&s_bar, (uint32_t)(rows * kn) * 4u);
        if (kn > 0)
            for (int r = 0; r < rows; ++r)
                tc::bulk_load(ws + (size_t)r * wstride, W + (size_t)(n0 + r) * K + k_lo, (uint32_t)kn * 4u, &s_bar);
    }
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // "I run": completes once all do
    pdl_wait();                 // everything below reads what earlier kernels of the step wrote
    pdl_launch();
    __syncthreads();            // the barrier is initialised

    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    const int nchunks = (kn + 7) / 8;
    float acc[MI][RJ];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < RJ; ++j) acc[i][j] = 0.f;
    // this lane's rows of x (tokens tg, tg + 8, ...), as offsets from the slice's start; a token beyond M reads token 0
    // and is never written
    const float* xs = x + k_lo;
    long long xoff[MI];
#pragma unroll
    for (int i = 0; i < MI; ++i) xoff[i] = (tg + 8 * i < M ? (long long)(tg + 8 * i) : 0LL) * ldx;
    float4 xa[MI][2], xb[MI][2];
    auto load_x = [&](int c, float4 (&dst)[MI][2]) {
        const bool h1 = c * 8 + 4 < kn;                   // the last chunk of a slice may hold 4 floats only
#pragma unroll
        for (int i = 0; i < MI; ++i) {
            const float* row = xs + xoff[i] + c * 8;
            dst[i][0] = __ldcg(reinterpret_cast<const float4*>(row));
            dst[i][1] = h1 ? __ldcg(reinterpret_cast<const float4*>(row + 4)) : zero4;
        }
    };
    auto multiply = [&](int c, const float4 (&xv)[MI][2]) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int k = c * 8 + 4 * h;
            if (k < kn) {
#pragma unroll
                for (int j = 0; j < RJ; ++j) {
                    const int r = rg + 4 * j;
                    const float4 w = r < rows ? *reinterpret_cast<const float4*>(ws + (size_t)r * wstride + k) : zero4;
#pragma unroll
                    for (int i = 0; i < MI; ++i) acc[i][j] = dot4(w, xv[i][h], acc[i][j]);
                }
            }
        }
    };
    if (warp < nchunks) load_x(warp, xa);
    const bool arrived = tc::mbar_wait(&s_bar, 0);
    if (!arrived && t == 0) {             // gave up: tell the host; the results of the step are not used
        atomicCAS(&g_stream_error, 0, 1);
        tc::report_to_host(402);
    }
    if (arrived) {
        // two chunks per round, the two register sets in turn: the next chunk's values are on their way while one is multiplied
        for (int c = warp; c < nchunks; c += 2 * WARPS) {
            if (c + WARPS < nchunks) load_x(c + WARPS, xb);
            multiply(c, xa);
            if (c + WARPS < nchunks) {
                if (c + 2 * WARPS < nchunks) load_x(c + 2 * WARPS, xa);
                multiply(c + WARPS, xb);
            }
        }
    }
    // the warps' partial tiles meet in shared memory
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < RJ; ++j) red[((size_t)warp * MT + tg + 8 * i) * rstride + rg + 4 * j] = acc[i][j];
    __syncthreads();
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // rank 0 runs: its memory may be written
    constexpr int PER = (MT * RT + WARPS * 32 - 1) / (WARPS * 32);        // outputs per thread
    float v[PER];
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int o = t + q * WARPS * 32;
        v[q] = 0.f;
        if (o < MT * RT) {
            const int m = o / RT, r = o % RT;
            float sum = red[(size_t)m * rstride + r];
#pragma unroll
            for (int w = 1; w < WARPS; ++w) sum += red[((size_t)w * MT + m) * rstride + r];     // warp order
            v[q] = sum;
            if (rank > 0) cluster.map_shared_rank(part, 0)[(size_t)(rank - 1) * MT * RT + o] = sum;
        }
    }
    if (S > 1) {
        cluster.sync();                                                        // every slice's tile is in place
        if (rank != 0) return;
    }
#pragma unroll
    for (int q = 0; q < PER; ++q) {
        const int o = t + q * WARPS * 32;
        const int m = o / RT, n = n0 + o % RT;
        if (o < MT * RT && m < M && n < N) {
            float sum = v[q];
            for (int p = 1; p < S; ++p) sum += part[(size_t)(p - 1) * MT * RT + o];               // rank order
            const bool to_cache = KVW && n >= kv.q_size;
            const float old = (accumulate && !to_cache) ? __ldcg(out + (size_t)m * ldo + n) : 0.f;
            const int slot = to_cache ? __ldcg(kv.slots + m) : 0;
            finish_one<KVW>(sum, m, n, bias ? __ldg(bias + n) : 0.f, out, ldo, act, accumulate, old, slot, kv);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Rows of W up to 2048 long, up to 64 rows of x (as many as fit shared memory): at most one CTA per SM, which stays
// and walks tiles of 32 weight rows (16 with 2 rows per warp); a warp owns 4 (2) rows of the tile and all of K, its
// lanes split K in float4 steps of 128.  The (normalised) rows of x are put into shared memory once per CTA; the
// weights come straight from HBM into registers, 4 rows x K in flight per warp, the first tile's before the kernel
// waits for its predecessor.  A value of x read from shared memory meets 4 weight rows (16 multiply-adds per
// 16-byte read, which keeps shared memory off the critical path), and the 32 sums of a lane meet inside the warp by
// the halving butterfly, after which lane 8r + m holds row r, token m: no barrier and no shared memory in the loop,
// and the norm's statistics once per SM instead of once per tile.  Per tile that is a third of the instructions of
// the kernel above, which at 50,257 rows is bound by its instructions, not by HBM, and which at the widths of GPT-2
// medium and XL needs two or three waves of CTAs.  With a Q|K|V matrix the key and value columns go to their slots.
template <int KP, int RW, bool LN, bool KVW>     // KP: float4 steps of K per lane (K <= KP * 128); RW: weight rows of a warp (4 or 2)
// (The narrow variant without the norm is held to 128 registers: two of its CTAs, or one and the CTAs of the next
// kernel, whose loads then start earlier, fit an SM; measured 0.5 us per block faster at 1 to 16 rows.  With the norm
// the cap costs more in the kernel than the earlier start brings.)
__global__ void __launch_bounds__(WARPS * 32, (KP == 8 && RW == 2 && !LN) ? 2 : 1)
linear_stream_f32_tall_kernel(const float* x, long long ldx, const float* __restrict__ W, const float* __restrict__ bias,
                              float* out, long long ldo, int M, int N, int K, int act, int accumulate, LnArgs ln,
                              KvArgs kv) {
    extern __shared__ __align__(16) float xs[];             // [M up to a multiple of 8][K up to a multiple of 128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int TR = WARPS * RW, V = RW * 8;             // rows of a tile; sums of a lane
    const int tiles = (N + TR - 1) / TR;
    float4 w[RW][KP];
    auto load_w = [&](int tile) {
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int n = tile * TR + warp * RW + r;
            const float* row = W + (size_t)(n < N ? n : 0) * K;
#pragma unroll
            for (int c = 0; c < KP; ++c) {
                const int k = c * 128 + lane * 4;
                w[r][c] = (k < K && n < N) ? __ldcs(reinterpret_cast<const float4*>(row + k)) : zero4;
            }
        }
    };
    int tile = blockIdx.x;
    if (tile < tiles) load_w(tile);          // weights depend on no kernel of the step
    pdl_wait();
    pdl_launch();
    const int KS = (K + 127) / 128 * 128;                   // a row of x in shared memory, its tail beyond K zero
    const int passes = (M + 7) / 8;
    for (int m = warp; m < passes * 8; m += WARPS) {   // a warp stages tokens warp, warp + 8, ... (normalised if asked for); rows beyond M are zero
        if (m >= M) {
#pragma unroll
            for (int c = 0; c < KP; ++c)
                if (c * 128 < K) *reinterpret_cast<float4*>(xs + (size_t)m * KS + c * 128 + lane * 4) = zero4;
            continue;
        }
        float4 rv[KP];
        const float* xbase = LN ? ln.x : x;
        const float* row = xbase + (size_t)((LN && ln.rows) ? __ldcg(ln.rows + m) : m) * ldx;
#pragma unroll
        for (int c = 0; c < KP; ++c) {
            const int k = c * 128 + lane * 4;
            rv[c] = k < K ? __ldcg(reinterpret_cast<const float4*>(row + k)) : zero4;
        }
        if constexpr (LN) {
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < KP; ++c) sum += (rv[c].x + rv[c].y) + (rv[c].z + rv[c].w);
            const float mean = warp_sum(sum) / (float)K;
            float var = 0.f;
#pragma unroll
            for (int c = 0; c < KP; ++c) {
                if (c * 128 + lane * 4 < K) {
                    const float a = rv[c].x - mean, b = rv[c].y - mean, cc = rv[c].z - mean, d = rv[c].w - mean;
                    var += (a * a + b * b) + (cc * cc + d * d);
                }
            }
            const float rstd = rsqrtf(warp_sum(var) / (float)K + ln.eps);
#pragma unroll
            for (int c = 0; c < KP; ++c) {
                const int k = c * 128 + lane * 4;
                if (k < K) {
                    const float4 g = __ldg(reinterpret_cast<const float4*>(ln.gamma + k));
                    const float4 b = __ldg(reinterpret_cast<const float4*>(ln.beta + k));
                    rv[c].x = (rv[c].x - mean) * rstd * g.x + b.x;
                    rv[c].y = (rv[c].y - mean) * rstd * g.y + b.y;
                    rv[c].z = (rv[c].z - mean) * rstd * g.z + b.z;
                    rv[c].w = (rv[c].w - mean) * rstd * g.w + b.w;
                }
            }
        }
#pragma unroll
        for (int c = 0; c < KP; ++c)
            if (c * 128 < K) *reinterpret_cast<float4*>(xs + (size_t)m * KS + c * 128 + lane * 4) = rv[c];   // zero beyond K
    }
    __syncthreads();
    for (; tile < tiles; tile += gridDim.x) {
        const int n_base = tile * TR + warp * RW;
        for (int p = 0; p < passes; ++p) {                   // 8 tokens at a time against the same registers of weights
            float acc[V];                                    // [row][token]
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.f;
            const int m0 = p * 8;
            // what the epilogue of this lane needs (bias, the old value or the cache slot) is fetched before the products
            const int e_v = V == 32 ? lane : lane >> 1;
            const int e_m = m0 + (e_v & 7), e_n = n_base + (e_v >> 3);
            const bool e_ok = e_m < M && e_n < N && (V == 32 || (lane & 1) == 0);
            float e_bias = 0.f, e_old = 0.f;
            int e_slot = 0;
            if (e_ok) {
                if (bias) e_bias = __ldg(bias + e_n);
                if (KVW && e_n >= kv.q_size) e_slot = __ldcg(kv.slots + e_m);
                else if (accumulate) e_old = __ldcg(out + (size_t)e_m * ldo + e_n);
            }
            const float* xp = xs + (size_t)m0 * KS + lane * 4;
            if (M - m0 > 4) {
                // all 8 rows of the pass without a branch between the reads (rows beyond M hold zeros)
#pragma unroll
                for (int c = 0; c < KP; ++c) {
                    if (c * 128 < K) {
#pragma unroll
                        for (int m = 0; m < 8; ++m) {
                            const float4 xv = *reinterpret_cast<const float4*>(xp + (size_t)m * KS + c * 128);
#pragma unroll
                            for (int r = 0; r < RW; ++r) acc[r * 8 + m] = dot4(w[r][c], xv, acc[r * 8 + m]);
                        }
                    }
                }
            } else if (M - m0 > 2) {                         // three or four rows: the first four
#pragma unroll
                for (int c = 0; c < KP; ++c) {
                    if (c * 128 < K) {
#pragma unroll
                        for (int m = 0; m < 4; ++m) {
                            const float4 xv = *reinterpret_cast<const float4*>(xp + (size_t)m * KS + c * 128);
#pragma unroll
                            for (int r = 0; r < RW; ++r) acc[r * 8 + m] = dot4(w[r][c], xv, acc[r * 8 + m]);
                        }
                    }
                }
            } else {                                         // one or two rows: only these
#pragma unroll
                for (int c = 0; c < KP; ++c) {
                    if (c * 128 < K) {
#pragma unroll
                        for (int m = 0; m < 2; ++m) {
                            if (m0 + m < M) {
                                const float4 xv = *reinterpret_cast<const float4*>(xp + (size_t)m * KS + c * 128);
#pragma unroll
                                for (int r = 0; r < RW; ++r) acc[r * 8 + m] = dot4(w[r][c], xv, acc[r * 8 + m]);
                            }
                        }
                    }
                }
            }
            // the next tile's weights fly while this one's sums meet (all loads in one burst: issued one column at
            // a time between the multiply-adds they were slower by half)
            if (p == passes - 1 && tile + (int)gridDim.x < tiles) load_w(tile + gridDim.x);
#pragma unroll
            for (int half = V / 2, off = 16; half >= 1; half >>= 1, off >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = upper ? acc[i] : acc[i + half];
                    const float keep = upper ? acc[i + half] : acc[i];
                    acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            if constexpr (V == 16) acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
            // the lane holds the sum of value v = 8 * row + token: v = lane with 32 sums, lane / 2 with 16
            if (e_ok) finish_one<KVW>(acc[0], e_m, e_n, e_bias, out, ldo, act, accumulate, e_old, e_slot, kv);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Rows of W longer than 2048 (a down-projection), up to 64 rows of x: the arrangement of the kernel above with K
// cut twice.  A CTA owns a tile of 32 weight rows (4 per warp) over a slice of K (the S CTAs of a thread-block
// cluster share a tile's K), and walks its slice in chunks of KP * 128 floats.  Per chunk the CTA puts all rows of
// x into shared memory once (asynchronous 16-byte copies), every warp holds its 4 x chunk weights in registers
// (straight from HBM; the first chunk's before the wait on the previous kernel, the next chunk's issued in one
// burst before the last sums of this one meet), and 8 tokens at a time go against them.  A lane's 32 sums meet
// inside the warp by the halving butterfly; lane 8r + m then holds row r, token m of the pass.  Chunks are added in
// chunk order (in shared memory), slices in rank order: rank q finishes the passes q, q + S, ... and reads the
// other slices' sums over the SM-to-SM network, all at once.
template <int KP, bool KVW>
__global__ void __launch_bounds__(WARPS * 32, KP <= 3 ? 2 : 1)
linear_stream_f32_regs_kernel(const float* x, long long ldx, const float* __restrict__ W, const float* __restrict__ bias,
                              float* out, long long ldo, int M, int N, int K, int Ls, int S, int act, int accumulate,
                              KvArgs kv) {
    constexpr int KC = KP * 128, RW = 4, TR = WARPS * RW;
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int passes = (M + 7) / 8;
    float* xs = smem;                                       // [passes * 8][KC]
    float* red = smem + (size_t)passes * 8 * KC;            // [passes][WARPS][32] sums over the chunks so far
    const int tile = blockIdx.x / S, rank = blockIdx.x % S;
    const int k_lo = min(K, rank * Ls), k_hi = min(K, k_lo + Ls);
    const int chunks = (k_hi - k_lo + KC - 1) / KC;         // 0: an empty slice adds nothing
    const int n_base = tile * TR + warp * RW;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 w[RW][KP];
    auto load_w = [&](int c) {
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int n = n_base + r;
            const float* row = W + (size_t)(n < N ? n : 0) * K;
#pragma unroll
            for (int col = 0; col < KP; ++col) {
                const int k = k_lo + c * KC + col * 128 + lane * 4;
                w[r][col] = (k < k_hi && n < N) ? __ldcs(reinterpret_cast<const float4*>(row + k)) : zero4;
            }
        }
    };
    if (chunks > 0) load_w(0);                // weights depend on no kernel of the step
    // after the butterfly the lane holds row e_r of the warp and token e_m of the pass; rank q finishes the passes
    // q, q + S, ... and fetches what their epilogue needs (the old value or the cache slot) long before
    const int e_r = lane >> 3, e_m = lane & 7, e_n = n_base + e_r;
    const bool e_col = e_n < N;
    const float e_bias = (e_col && bias) ? __ldg(bias + e_n) : 0.f;
    pdl_wait();
    pdl_launch();
    float e_old[8];
    int e_slot[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = (rank + i * S) * 8 + e_m;
        e_old[i] = 0.f;
        e_slot[i] = 0;
        if (e_col && m < M) {
            if (KVW && e_n >= kv.q_size) e_slot[i] = __ldcg(kv.slots + m);
            else if (accumulate) e_old[i] = __ldcg(out + (size_t)m * ldo + e_n);
        }
    }
    const bool direct = S == 1 && chunks == 1;     // the sums go out as they meet
    const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);
    for (int c = 0; c < chunks; ++c) {
        if (c > 0) __syncthreads();                // the chunk before has been read by every warp
        const int kc0 = k_lo + c * KC;
        // rows of x into shared memory by asynchronous 16-byte copies (zeros beyond M and beyond the slice)
        for (int m = warp; m < passes * 8; m += WARPS) {
#pragma unroll
            for (int col = 0; col < KP; ++col) {
                const int k = kc0 + col * 128 + lane * 4;
                const bool in = m < M && k < k_hi;
                const float* src = in ? x + (size_t)m * ldx + k : x;
                const uint32_t dst = xs_addr + (uint32_t)(((size_t)m * KC + col * 128 + lane * 4) * 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(in ? 16 : 0) : "memory");
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        const int len = min(KC, k_hi - kc0);
#pragma unroll 1
        for (int p = 0; p < passes; ++p) {
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.f;
            const float* xp = xs + (size_t)p * 8 * KC + lane * 4;
            const int rows = M - p * 8;                       // rows of x in this pass (8 or more: all 8)
            if (rows > 4) {
#pragma unroll
                for (int col = 0; col < KP; ++col) {
                    if (col * 128 < len) {
#pragma unroll
                        for (int m = 0; m < 8; ++m) {
                            const float4 xv = *reinterpret_cast<const float4*>(xp + (size_t)m * KC + col * 128);
#pragma unroll
                            for (int r = 0; r < RW; ++r) acc[r * 8 + m] = dot4(w[r][col], xv, acc[r * 8 + m]);
                        }
                    }
                }
            } else {                                          // up to four rows: the first two, then the next two if any
#pragma unroll
                for (int col = 0; col < KP; ++col) {
                    if (col * 128 < len) {
#pragma unroll
                        for (int m = 0; m < 4; ++m) {
                            if (m < 2 || rows > 2) {
                                const float4 xv = *reinterpret_cast<const float4*>(xp + (size_t)m * KC + col * 128);
#pragma unroll
                                for (int r = 0; r < RW; ++r) acc[r * 8 + m] = dot4(w[r][col], xv, acc[r * 8 + m]);
                            }
                        }
                    }
                }
            }
            if (p == passes - 1 && c + 1 < chunks) load_w(c + 1);
#pragma unroll
            for (int half = 16, off = 16; half >= 1; half >>= 1, off >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = upper ? acc[i] : acc[i + half];
                    const float keep = upper ? acc[i + half] : acc[i];
                    acc[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            if (direct) {
                const int m = p * 8 + e_m;
                float old = 0.f;
                int sl = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i == p) old = e_old[i], sl = e_slot[i];
                if (e_col && m < M) finish_one<KVW>(acc[0], m, e_n, e_bias, out, ldo, act, accumulate, old, sl, kv);
            } else {
                float* slot = red + ((size_t)p * WARPS + warp) * 32 + lane;
                *slot = c == 0 ? acc[0] : *slot + acc[0];      // only this lane touches the slot
            }
        }
    }
    if (direct) return;
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) cluster.sync();                                 // every slice's sums are in place
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int p = rank + i * S;
        if (p < passes) {
            const size_t at = ((size_t)p * WARPS + warp) * 32 + lane;
            float part[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {                      // all slices' sums on their way at once
                part[q] = 0.f;
                if (q < S && q * Ls < K) part[q] = S > 1 ? cluster.map_shared_rank(red, q)[at] : red[at];
            }
            float v = part[0];
#pragma unroll
            for (int q = 1; q < 8; ++q)
                if (q < S) v += part[q];                       // rank order
            const int m = p * 8 + e_m;
            if (e_col && m < M) finish_one<KVW>(v, m, e_n, e_bias, out, ldo, act, accumulate, e_old[i], e_slot[i], kv);
        }
    }
    if (S > 1) cluster.sync();                                 // the others' shared memory has been read
}

// Rows of x that the kernel above takes at a width K: what fits its shared memory, in eights, 64 at most (a function
// of K alone, so that which kernel sums a row does not depend on the batch beyond that)
constexpr int TALL_SMEM_LIMIT = 216 * 1024;
int tall_rows(int K) {
    if (K > 2048) return 0;
    const int fit = TALL_SMEM_LIMIT / ((K + 127) / 128 * 128 * 4) / 8 * 8;
    return fit < MAX_M ? fit : MAX_M;
}

int sm_count();
// K slices with which the kernel for long rows takes M rows of x against a matrix [N, K] (0: another kernel does).
// From the matrix alone, except for the side of 16 rows.  Measured at the down-projections of GPT-2 small, medium
// and XL against the tile kernels: with the largest of 4 or 2 slices whose CTAs fit the SMs at once it wins at every
// row count where the chunks of 768 fill the slice to 4/5 at least (768 x 3072 in 4 slices: 5.0 / 5.1 / 7.0 us at
// 1 / 8 / 16 rows against 5.6 / 5.9 / 9.4 us, 17.9 against 19.0 us at 64; 1600 x 6400 in 2 slices: 16 against 20 us at
// 8 rows, 72 against 92 us at 64); where they do not (1024 x 4096: slices of 1024 are a chunk and a third) it loses
// up to 16 rows (7.8 against 7.2 us) and wins beyond (27 against 32 us at 64).
constexpr int REGS_KC = 768;
int regs_slices(int N, int K, int M) {
    if (K <= 2048 || K % 4 != 0) return 0;
    const int tiles = (N + 31) / 32, sms = sm_count();
    int S = tiles * 4 <= sms ? 4 : tiles * 2 <= sms ? 2 : 0;
    if (!S) return 0;
    const int Ls = ((K + S - 1) / S + 127) / 128 * 128;
    const int chunks = (Ls + REGS_KC - 1) / REGS_KC;
    const bool filled = 4 * chunks * REGS_KC <= 5 * Ls;
    return (filled || M > FEW_M) ? S : 0;
}

// Whether the kernel above takes a matrix, and with how many weight rows per warp (0: not this kernel), from the
// matrix alone.  Measured against the tile kernels at the layer shapes of GPT-2 small, medium and XL and 1, 8 and 16
// rows of x: up to K = 1024 it wins everywhere (3.4-6 us against 3.9-8.5 us), with 4 rows per warp once those
// tiles of 32 rows fill more than half of the SMs, else with 2; from K = 1025 to 2048 it wins when its tiles of 16
// rows fill the SMs at least once (N >= 2368 on 148 SMs: 14 against 25 us at 4800 x 1600), and loses for narrower
// matrices (6.8 against 5.3 us at 1600 x 1600), where the tile kernel's K slices keep more SMs busy.
int tall_shape(int N, int K) {
    if (K > 2048) return 0;
    const int sms = sm_count();
    if (K <= 1024) return 5 * ((N + 31) / 32) >= 3 * sms ? 4 : 2;
    return (N + 15) / 16 >= sms ? 2 : 0;
}
// Rows of x up to which it is taken: all that fit shared memory for a matrix as tall as a vocabulary; 48 with 4 weight
// rows per warp (3072 x 768 at 48 rows: 20.9 against 22.1 us of the kernel for 17 to 64 rows, 3072 x 1024: 24.6
// against 29.4 us; at 64 rows they are even or it loses), 24 with K over 1024 (4800 x 1600 at 24 rows: 38.5 against
// 42.9 us, at 32 rows 49.2 against 45.4 us), 16 for narrower matrices (2304 x 768 at 24 rows: 13.0 against 12.4 us).
int tall_rows_for(int N, int K) {
    const int rw = tall_shape(N, K);
    if (!rw) return 0;
    const int fit = tall_rows(K);
    if ((N + 31) / 32 >= 8 * sm_count()) return fit;
    const int cap = K > 1024 ? 24 : (rw == 4 ? 48 : FEW_M);
    return fit < cap ? fit : cap;
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
// rows gets slices while its CTAs still fit the GPU in one wave of two per SM and a slice keeps at least 256 of K.
MLLM_EXPORT int mllm_linear_stream_f32_slices(int N, int K) {
    int S = 1;
    const int tiles = (N + R - 1) / R;
    while (S < MAX_SLICES && tiles * S * 2 <= 2 * sm_count() && K / (2 * S) >= 256) S *= 2;
    return S;
}

constexpr size_t MANY_SMEM_LIMIT = 200 * 1024;
size_t many_smem_bytes(int RT, int Ks, int S, int MT) {
    return ((size_t)RT * (Ks + MANY_WS_PAD) + (size_t)WARPS * MT * (RT + MANY_RED_PAD) + (S > 1 ? (size_t)(S - 1) * MT * RT : 0)) * 4;
}

// Tile height (16, 24 or 32 weight rows) and K slices (1, 2, 4 or 8 CTAs of a cluster) of the kernel for 17 to 64 rows,
// from the matrix alone (never from M): the pair with the least estimated time, waves of CTAs (one CTA per SM) times a
// CTA's work, its tile's RT x Ks products plus a fixed cost of meeting, reducing and finishing worth about 32 x 256 of
// them; among equals the taller tile (it reads x less often), then fewer slices.  A slice keeps at least 192 of K.
MLLM_EXPORT int mllm_linear_stream_f32_many_shape(int N, int K, int* rt, int* slices) {
    const int sms = sm_count();
    int best_rt = 32, best_s = 1;
    long long best = -1;
    for (int RT = 32; RT >= 16; RT -= 8)
        for (int S = 1; S <= 8; S *= 2) {
            if (S > 1 && K / S < 192) break;
            const long long ks = ((K + S - 1) / S + 3) / 4 * 4;
            if (many_smem_bytes(RT, (int)ks, S, MAX_M) > MANY_SMEM_LIMIT) continue;     // (for 64 rows: the choice must not depend on M)
            const long long ctas = (long long)((N + RT - 1) / RT) * S;
            const long long waves = (ctas + sms - 1) / sms;
            const long long cost = waves * ((long long)RT * ks + 8192);
            if (best < 0 || cost < best) best = cost, best_rt = RT, best_s = S;
        }
    *rt = best_rt;
    *slices = best_s;
    return best < 0 ? 1 : 0;        // 1: no shape fits shared memory (K beyond about 48,000): the caller takes another kernel
}

// Rows of x up to which a matrix [N, K] goes to the kernel with the weights in registers (0: never).
MLLM_EXPORT int mllm_linear_stream_f32_tall_rows(int N, int K) { return tall_rows_for(N, K); }

// Which kernel of this file computes M plain rows (no norm, no cache write) against a matrix [N, K]: 0 threads split K
// (up to 16 rows), 1 warps own tokens (17 to 64 rows), 2 weights in registers, 3 long rows in cluster slices.  Rows
// computed by the same kernel have the same bits whatever the batch.
MLLM_EXPORT int mllm_linear_stream_f32_kernel_of(int M, int N, int K) {
    if (M <= tall_rows_for(N, K)) return 2;
    if (regs_slices(N, K, M)) return 3;
    return M <= FEW_M ? 0 : 1;
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
    LnArgs ln = {(const float*)ln_x, ln_rows, ln_gamma, ln_beta, ln_eps};
    KvArgs kv = {(float*)k_pages, (float*)v_pages, slots, q_size, kv_heads, head_dim, page_size};
    const int tiles = (N + R - 1) / R;
    const int tall_rw = M <= tall_rows_for(N, K) ? tall_shape(N, K) : 0;
    if (tall_rw) {
        // weights from HBM into registers, x in shared memory once per CTA, CTAs that stay and walk the tiles
        const size_t smem = (size_t)((M + 7) / 8 * 8) * ((K + 127) / 128 * 128) * 4;
        using Tall = void (*)(const float*, long long, const float*, const float*, float*, long long, int, int, int, int, int,
                              LnArgs, KvArgs);
        const int shape = K > 1024 ? 2 : (tall_rw == 2 ? 1 : 0);
        const int which = shape * 4 + (norm ? 2 : 0) + (kvw ? 1 : 0);
#define MLLM_TALL(KP, RW) linear_stream_f32_tall_kernel<KP, RW, false, false>, linear_stream_f32_tall_kernel<KP, RW, false, true>, \
                          linear_stream_f32_tall_kernel<KP, RW, true, false>, linear_stream_f32_tall_kernel<KP, RW, true, true>
        static const Tall kerns[12] = {MLLM_TALL(8, 4), MLLM_TALL(8, 2), MLLM_TALL(16, 2)};
#undef MLLM_TALL
        static bool wide[12] = {};
        if (smem > 48 * 1024 && !wide[which]) {
            MLLM_CUDA(cudaFuncSetAttribute(kerns[which], cudaFuncAttributeMaxDynamicSharedMemorySize, TALL_SMEM_LIMIT));
            wide[which] = true;
        }
        const int rows_tile = WARPS * (shape == 0 ? 4 : 2);
        const int tiles_tall = (N + rows_tile - 1) / rows_tile;
        const int grid = tiles_tall < sm_count() ? tiles_tall : sm_count();
        MLLM_CUDA(mllm_launch(kerns[which], dim3(grid), dim3(WARPS * 32), smem, stream, true, (const float*)x, ldx,
                              (const float*)W, bias, (float*)out, ldo, M, N, K, act, accumulate, ln, kv));
        return 0;
    }
    const int regs_s = regs_slices(N, K, M);
    if (regs_s && !norm && !kvw) {
        // long rows: K slices in a cluster, chunks in registers
        const int S = regs_s;
        const int Ls = ((K + S - 1) / S + 127) / 128 * 128;
        const size_t smem = ((size_t)((M + 7) / 8 * 8) * REGS_KC + (size_t)((M + 7) / 8) * WARPS * 32) * 4;
        auto kern = linear_stream_f32_regs_kernel<REGS_KC / 128, false>;
        static bool wide_regs = false;
        if (smem > 48 * 1024 && !wide_regs) {
            MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (MAX_M * REGS_KC + MAX_M / 8 * WARPS * 32) * 4));
            wide_regs = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((N + 31) / 32 * S);
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
        MLLM_CUDA(cudaLaunchKernelEx(&cfg, kern, (const float*)x, ldx, (const float*)W, bias, (float*)out, ldo, M, N, K, Ls, S,
                                     act, accumulate, kv));
        return 0;
    }
    if (M <= FEW_M) {
        // threads split K; CTAs own several tiles of narrow K so that the grid is one wave of two CTAs per SM
        int S = norm ? 1 : mllm_linear_stream_f32_slices(N, K);
        int Ks = ((K + S - 1) / S + 3) / 4 * 4;
        while (!norm && S < MAX_SLICES && (size_t)R * Ks * 4 > 96 * 1024) {       // rows too long for shared memory
            S *= 2;
            Ks = ((K + S - 1) / S + 3) / 4 * 4;
        }
        int T = 1;
        if (S == 1)      // measured: two CTAs per SM in one wave beat one CTA per SM with twice the tiles
            while (T < MAX_TILES && (tiles + T - 1) / T > 2 * sm_count() && (size_t)(T + 1) * R * Ks * 4 <= 96 * 1024) ++T;
        const size_t smem = ((size_t)T * R * Ks + 2 * WARPS * 64 + (S > 1 ? S * 128 : 0)) * 4;
        if (smem > 200 * 1024) return mllm_fail(1, "linear_stream_f32: K=%d is too long for shared memory", K);
        using Few = void (*)(const float*, long long, const float*, const float*, float*, long long, int, int, int, int,
                             int, int, int, int, LnArgs, KvArgs);
        Few kern = norm ? (kvw ? (Few)linear_stream_f32_few_kernel<true, true> : (Few)linear_stream_f32_few_kernel<true, false>)
                        : (kvw ? (Few)linear_stream_f32_few_kernel<false, true> : (Few)linear_stream_f32_few_kernel<false, false>);
        if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((tiles + T - 1) / T * S);
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
        MLLM_CUDA(cudaLaunchKernelEx(&cfg, kern, (const float*)x, ldx, (const float*)W, bias, (float*)out, ldo, M, N, K, Ks,
                                     S, T, act, accumulate, ln, kv));
        return 0;
    }
    // 17 to 64 rows: tile height and K slices from (N, K) alone, so that the CTAs fill the SMs once as fully as possible
    int RT = 32, S = 1;
    if (mllm_linear_stream_f32_many_shape(N, K, &RT, &S))
        return mllm_fail(1, "linear_stream_f32: K=%d is too long for shared memory", K);
    const int Ks = ((K + S - 1) / S + 3) / 4 * 4;
    const int MT = M <= 32 ? 32 : 64;
    const size_t smem = many_smem_bytes(RT, Ks, S, MT);
    using Many = void (*)(const float*, long long, const float*, const float*, float*, long long, int, int, int, int, int,
                          int, int, KvArgs);
    Many kern = nullptr;
#define PICK(I, J)                                                                                                   \
    if (MT == 8 * I && RT == 4 * J)                                                                                  \
        kern = kvw ? (Many)linear_stream_f32_many_kernel<I, J, true> : (Many)linear_stream_f32_many_kernel<I, J, false>;
    PICK(4, 4) PICK(4, 6) PICK(4, 8) PICK(8, 4) PICK(8, 6) PICK(8, 8)
#undef PICK
    if (!kern) return mllm_fail(1, "linear_stream_f32: no kernel for M=%d, %d rows per tile", M, RT);
    if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + RT - 1) / RT * S);
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
                                 act, accumulate, kv));
    return 0;
}
