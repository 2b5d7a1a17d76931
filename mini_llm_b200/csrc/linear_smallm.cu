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
    return __ldcg(reinterpret_cast<const uint4*>(p));     // the previous kernel's output: past L1, never the non-coherent path
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Fused LayerNorm on the input (x is then the 32-bit residual stream, optionally gathered by
// `rows`): every CTA computes mean and 1/std of its M rows itself (M <= 64 rows of K floats
// from L2) and normalises the values as it loads them, rounding to bfloat16 exactly where a
// separate norm kernel would have stored them.
struct NormArgs {
    const float* x;          // [*, K] 32-bit, row stride ldx
    const int* rows;         // optional gather
    const float* gamma;
    const float* beta;
    float eps;
};
// Fused cache write on the output of a Q|K|V projection: columns [0, q_size) go to q_out,
// the key and value columns go straight to their page slots
// ([page][kv_head][offset][head_dim], slot = page * page_size + offset).
struct KvArgs {
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    const int* slots;
    int q_size, kv_heads, head_dim, page_size;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int MT, int RT_, typename TO, bool LN, bool KVW>
__global__ void __launch_bounds__(WARPS * 32)
linear_smallm_kernel(const __nv_bfloat16* x, long long ldx, const __nv_bfloat16* __restrict__ W,
                     const float* __restrict__ bias, TO* out, long long ldo, int M, int N, int K, int act,
                     int accumulate, NormArgs ln, KvArgs kv) {
    // RT_ == 0 stands for half a row tile: 8 weight rows per CTA (the upper half of the MMA's 16 rows
    // stays zero), which doubles the number of CTAs for narrow matrices.
    constexpr bool HALF = RT_ == 0;
    constexpr int RT = HALF ? 1 : RT_;
    extern __shared__ float red[];                 // [WARPS][ROWS][8*MT], then the normed rows (LN)
    __shared__ float s_mean[LN ? 64 : 1], s_rstd[LN ? 64 : 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    constexpr int U = HALF ? 8 : (RT == 1 ? 4 : (RT == 2 ? 2 : 1));
    constexpr int ROWS = HALF ? 8 : 16 * RT, COLS = 8 * MT;
    const int n0 = blockIdx.x * ROWS;
    const int nchunks = (K + 31) / 32;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    // normed rows in shared memory (bfloat16, rows padded by 8 so that 16-byte reads of 8 rows do not collide)
    const int xs_stride = K + 8;
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(red + WARPS * ROWS * COLS);
    const bool ln_smem = LN && K <= 1024;

    // The weight loads of the first round go out before anything else: they come from HBM and
    // nothing they need depends on the norm statistics or on the epilogue's operands.
    uint4 wa[U][RT], wb[U][RT], wa_next[U][RT], wb_next[U][RT];
    auto load_w = [&](int c0, uint4 (&da)[U][RT], uint4 (&db)[U][RT]) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (c0 + u * WARPS) * 32 + 8 * t;
            const bool kok = k < K;                 // K is a multiple of 8: a lane's 8 values are in or out together
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                const int ra = n0 + r * 16 + g, rb = ra + 8;
                da[u][r] = (kok && ra < N) ? ldg16(W + (size_t)ra * K + k) : zero;
                db[u][r] = (!HALF && kok && rb < N) ? ldg16(W + (size_t)rb * K + k) : zero;
            }
        }
    };
    load_w(warp, wa, wb);
    const bool two_rounds = warp + WARPS * U < nchunks;
    if (two_rounds) load_w(warp + WARPS * U, wa_next, wb_next);     // a second round too: K up to 2 x 32 x WARPS x U needs no load after the wait
    if constexpr (LN) {
        // gamma and beta are weights as well: into shared memory now, so that normalising costs no trip to L2 later
        if (ln_smem) {
            float* gb = reinterpret_cast<float*>(xs + (size_t)M * xs_stride);
            for (int k = threadIdx.x * 4; k < K; k += WARPS * 32 * 4) {
                *reinterpret_cast<float4*>(gb + k) = __ldg(reinterpret_cast<const float4*>(ln.gamma + k));
                *reinterpret_cast<float4*>(gb + K + k) = __ldg(reinterpret_cast<const float4*>(ln.beta + k));
            }
        }
    }
    pdl_wait();                 // everything below reads what earlier kernels of the step wrote
    pdl_launch();
    if constexpr (LN) {
        if (ln_smem) __syncthreads();               // gamma and beta are in shared memory for every warp
    }

    // The epilogue's operands of this thread's first output element, fetched early as well.
    const int e_row = threadIdx.x % ROWS, e_col = threadIdx.x / ROWS;
    const int e_n = n0 + e_row;
    const bool e_ok = threadIdx.x < ROWS * COLS && e_n < N && e_col < M;
    float e_bias = 0.f, e_old = 0.f;
    int e_slot = 0;
    if (e_ok) {
        if (bias) e_bias = bias[e_n];
        if (KVW && e_n >= kv.q_size) e_slot = kv.slots[e_col];
        else if (accumulate) e_old = to_f32(out[(size_t)e_col * ldo + e_n]);
    }

    if constexpr (LN) {
        // mean and 1/std of every row: one pass over the row in registers when it is short enough
        constexpr int KEEP = 8;                      // float4 per lane kept: rows up to 1024 wide
        for (int m = warp; m < M; m += WARPS) {
            const float* xr = ln.x + (size_t)(ln.rows ? ln.rows[m] : m) * ldx;
            float4 keep[KEEP];
            const bool fits = K <= KEEP * 128;
            float s = 0.f;
            if (fits) {
#pragma unroll
                for (int i = 0; i < KEEP; ++i) {
                    const int k = lane * 4 + i * 128;
                    keep[i] = k < K ? *reinterpret_cast<const float4*>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                    s += (keep[i].x + keep[i].y) + (keep[i].z + keep[i].w);
                }
            } else {
                for (int k = lane * 4; k < K; k += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(xr + k);
                    s += (v.x + v.y) + (v.z + v.w);
                }
            }
            const float mean = warp_sum(s) / (float)K;
            float q = 0.f;
            if (fits) {
#pragma unroll
                for (int i = 0; i < KEEP; ++i) {
                    if (lane * 4 + i * 128 < K) {
                        const float a = keep[i].x - mean, b = keep[i].y - mean, c = keep[i].z - mean, d = keep[i].w - mean;
                        q += (a * a + b * b) + (c * c + d * d);
                    }
                }
            } else {
                for (int k = lane * 4; k < K; k += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(xr + k);
                    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
                    q += (a * a + b * b) + (c * c + d * d);
                }
            }
            const float var = warp_sum(q) / (float)K;
            const float rstd = rsqrtf(var + ln.eps);
            if (lane == 0) { s_mean[m] = mean; s_rstd[m] = rstd; }
            if (fits) {
                // the normed row, rounded to bfloat16 as a separate norm kernel would store it
#pragma unroll
                for (int i = 0; i < KEEP; ++i) {
                    const int k = lane * 4 + i * 128;
                    if (k < K) {
                        const float* gb = reinterpret_cast<const float*>(xs + (size_t)M * xs_stride);   // staged before the wait (fits: K <= 1024)
                        const float4 ga = *reinterpret_cast<const float4*>(gb + k);
                        const float4 be = *reinterpret_cast<const float4*>(gb + K + k);
                        uint2 pk;
                        pk.x = pack2((keep[i].x - mean) * rstd * ga.x + be.x, (keep[i].y - mean) * rstd * ga.y + be.y);
                        pk.y = pack2((keep[i].z - mean) * rstd * ga.z + be.z, (keep[i].w - mean) * rstd * ga.w + be.w);
                        *reinterpret_cast<uint2*>(xs + (size_t)m * xs_stride + k) = pk;
                    }
                }
            }
        }
        __syncthreads();
    }

    float acc[RT][MT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[r][m][i] = 0.f;

    for (int c0 = warp; c0 < nchunks; c0 += WARPS * U) {
        const bool more = c0 + WARPS * U < nchunks;
        if (more && c0 != warp) load_w(c0 + WARPS * U, wa_next, wb_next);     // the next round's weights fly while this one is used (the second round went out before the wait)
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (c0 + u * WARPS) * 32 + 8 * t;
            const bool kok = k < K;
            uint4 xv[MT];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int row = m * 8 + g;
                xv[m] = zero;
                if (kok && row < M) {
                    if (ln_smem) {
                        xv[m] = *reinterpret_cast<const uint4*>(xs + (size_t)row * xs_stride + k);
                    } else if constexpr (LN) {
                        const float* xr = ln.x + (size_t)(ln.rows ? ln.rows[row] : row) * ldx + k;
                        const float4 a = *reinterpret_cast<const float4*>(xr), b = *reinterpret_cast<const float4*>(xr + 4);
                        const float4 ga = __ldg(reinterpret_cast<const float4*>(ln.gamma + k));
                        const float4 gb = __ldg(reinterpret_cast<const float4*>(ln.gamma + k + 4));
                        const float4 ba = __ldg(reinterpret_cast<const float4*>(ln.beta + k));
                        const float4 bb = __ldg(reinterpret_cast<const float4*>(ln.beta + k + 4));
                        const float mu = s_mean[row], rs = s_rstd[row];
                        xv[m].x = pack2((a.x - mu) * rs * ga.x + ba.x, (a.y - mu) * rs * ga.y + ba.y);
                        xv[m].y = pack2((a.z - mu) * rs * ga.z + ba.z, (a.w - mu) * rs * ga.w + ba.w);
                        xv[m].z = pack2((b.x - mu) * rs * gb.x + bb.x, (b.y - mu) * rs * gb.y + bb.y);
                        xv[m].w = pack2((b.z - mu) * rs * gb.z + bb.z, (b.w - mu) * rs * gb.w + bb.w);
                    } else {
                        xv[m] = ldg16_cached(x + (size_t)row * ldx + k);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < RT; ++r)
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    mma_bf16(acc[r][m], wa[u][r].x, wb[u][r].x, wa[u][r].y, wb[u][r].y, xv[m].x, xv[m].y);
                    mma_bf16(acc[r][m], wa[u][r].z, wb[u][r].z, wa[u][r].w, wb[u][r].w, xv[m].z, xv[m].w);
                }
        }
        if (more) {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < RT; ++r) { wa[u][r] = wa_next[u][r]; wb[u][r] = wb_next[u][r]; }
        }
    }
    // partial sums of this warp -> shared memory
    float* mine = red + (size_t)warp * ROWS * COLS;
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int row = r * 16 + g, col = m * 8 + 2 * t;
            mine[row * COLS + col] = acc[r][m][0];
            mine[row * COLS + col + 1] = acc[r][m][1];
            if constexpr (!HALF) {
                mine[(row + 8) * COLS + col] = acc[r][m][2];
                mine[(row + 8) * COLS + col + 1] = acc[r][m][3];
            }
        }
    __syncthreads();
    // consecutive threads take consecutive weight rows (n) of one token, so stores run along n
    for (int i = threadIdx.x; i < ROWS * COLS; i += WARPS * 32) {
        const int row = i % ROWS, col = i / ROWS;
        const int n = n0 + row;
        if (n >= N || col >= M) continue;
        const bool first = i == threadIdx.x;           // operands already in registers
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[(size_t)w * ROWS * COLS + row * COLS + col];
        if (bias) v += first ? e_bias : bias[n];
        v = (act == MLLM_ACT_GELU_TANH && sizeof(TO) == 2) ? gelu_tanh_fast(v) : apply_act(v, act);
        if constexpr (KVW) {
            if (n >= kv.q_size) {
                const int slot = first ? e_slot : kv.slots[col];
                if (slot < 0) continue;
                const int c = n - kv.q_size, kvs = kv.kv_heads * kv.head_dim;
                const int which = c / kvs, cc = c % kvs;
                const int head = cc / kv.head_dim, d = cc % kv.head_dim;
                const size_t dst = (((size_t)(slot / kv.page_size) * kv.kv_heads + head) * kv.page_size +
                                    slot % kv.page_size) * kv.head_dim + d;
                (which == 0 ? kv.k_pages : kv.v_pages)[dst] = __float2bfloat16_rn(v);
                continue;
            }
        }
        TO* o = out + (size_t)col * ldo + n;
        if (accumulate) v += first ? e_old : to_f32(*o);
        *o = from_f32<TO>(v);
    }
}

struct Call {
    const void* x; long long ldx; const void* W; const float* bias; void* out; long long ldo;
    int M, N, K, act, accumulate;
    const NormArgs* ln;       // null: plain bfloat16 input
    const KvArgs* kv;         // null: plain output
    cudaStream_t stream;
};

template <int MT, int RT, typename TO, bool LN, bool KVW>
int launch_k(const Call& c) {
    constexpr int ROWS = RT == 0 ? 8 : 16 * RT;
    size_t smem = (size_t)WARPS * ROWS * 8 * MT * sizeof(float);
    if (LN && c.K <= 1024) smem += (size_t)c.M * (c.K + 8) * sizeof(__nv_bfloat16) + 2 * (size_t)c.K * sizeof(float);   // the normed rows, gamma and beta
    auto kern = linear_smallm_kernel<MT, RT, TO, LN, KVW>;
    if (smem > 48 * 1024) {
        static size_t set = 0;                     // per instantiation: the largest size asked for so far
        if (smem > set) {
            MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            set = smem;
        }
    }
    const int grid = (c.N + ROWS - 1) / ROWS;
    MLLM_CUDA(mllm_launch(kern, dim3(grid), dim3(WARPS * 32), smem, c.stream, true, (const __nv_bfloat16*)c.x, c.ldx,
                          (const __nv_bfloat16*)c.W, c.bias, (TO*)c.out, c.ldo, c.M, c.N, c.K, c.act, c.accumulate,
                          c.ln ? *c.ln : NormArgs{}, c.kv ? *c.kv : KvArgs{}));
    return 0;
}

template <int MT, int RT, typename TO>
int pick_fusion(const Call& c) {
    if (c.kv) {
        if constexpr (sizeof(TO) == 2) {
            if (c.ln) return launch_k<MT, RT, TO, true, true>(c);
            return launch_k<MT, RT, TO, false, true>(c);
        } else {
            return mllm_fail(1, "linear_smallm: the cache-writing epilogue produces bfloat16");
        }
    }
    if (c.ln) return launch_k<MT, RT, TO, true, false>(c);
    return launch_k<MT, RT, TO, false, false>(c);
}

template <int MT, typename TO>
int pick_rt(int rt, const Call& c) {
    if (rt == 4) return pick_fusion<MT, 4, TO>(c);
    if (rt == 2) return pick_fusion<MT, 2, TO>(c);
    if (rt == 0) return pick_fusion<MT, 0, TO>(c);
    return pick_fusion<MT, 1, TO>(c);
}

template <typename TO>
int pick_mt(int rt, const Call& c) {
    if (c.M <= 8) return pick_rt<1, TO>(rt, c);
    if (c.M <= 16) return pick_rt<2, TO>(rt, c);
    if (c.M <= 32) return pick_rt<4, TO>(rt, c);
    return pick_rt<8, TO>(rt, c);
}

int dispatch(const Call& c, int out_dtype) {
    if (c.M <= 0 || c.N <= 0) return 0;
    if (c.M > 64) return mllm_fail(1, "linear_smallm: M=%d exceeds 64", c.M);
    if (c.K <= 0 || c.K % 8 != 0) return mllm_fail(1, "linear_smallm: K=%d is not a multiple of 8", c.K);
    if ((uintptr_t)c.W % 16 != 0) return mllm_fail(1, "linear_smallm: the weight must be 16-byte aligned");
    if (c.ln) {
        if (c.ldx % 4 != 0 || (uintptr_t)c.ln->x % 16 != 0 || (uintptr_t)c.ln->gamma % 16 != 0 ||
            (uintptr_t)c.ln->beta % 16 != 0)
            return mllm_fail(1, "linear_smallm: the normed input, gamma and beta must be 16-byte aligned");
    } else if (c.ldx % 8 != 0 || (uintptr_t)c.x % 16 != 0) {
        return mllm_fail(1, "linear_smallm: the input must be 16-byte aligned");
    }
    if (c.kv && (c.N != c.kv->q_size + 2 * c.kv->kv_heads * c.kv->head_dim || c.kv->page_size <= 0))
        return mllm_fail(1, "linear_smallm: %d output columns do not split into %d query and 2 x %d x %d cache columns",
                         c.N, c.kv->q_size, c.kv->kv_heads, c.kv->head_dim);
    // rows per CTA: enough CTAs to fill the 148 SMs when N allows it
    int rt = 1;
    if (c.N >= 16 * 4 * 296) rt = 4;
    else if (c.N >= 16 * 2 * 296) rt = 2;
    else if (c.N < 16 * 100 && c.M <= 16) rt = 0;   // narrow, few rows: 8 weight rows per CTA
    if (out_dtype == MLLM_BF16) return pick_mt<__nv_bfloat16>(rt, c);
    if (out_dtype == MLLM_F32) return pick_mt<float>(rt, c);
    return mllm_fail(1, "linear_smallm: unknown dtype code %d", out_dtype);
}

}  // namespace

// bfloat16 x and W; out bfloat16 or 32-bit.  Needs M <= 64, K a multiple of 8, and x
// and W 16-byte aligned with a row stride of x that is a multiple of 8.
MLLM_EXPORT int mllm_linear_smallm(const void* x, long long ldx, const void* W, const float* bias, void* out,
                                   long long ldo, int M, int N, int K, int act, int accumulate, int out_dtype,
                                   cudaStream_t stream) {
    Call c{x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, nullptr, nullptr, stream};
    return dispatch(c, out_dtype);
}

// The same product with LayerNorm fused on the input and/or the cache write fused on the
// output.  norm_x != null: the input is LayerNorm(norm_x[rows[m] or m]) with gamma, beta,
// eps (32-bit rows of K floats, row stride ldx, which is then counted in floats; `x` is
// ignored).  k_pages != null: columns >= q_size are keys then values and go to their page
// slots (bfloat16); `out` receives the first q_size columns only.
MLLM_EXPORT int mllm_linear_smallm_fused(const void* x, long long ldx, const void* W, const float* bias, void* out,
                                         long long ldo, int M, int N, int K, int act, int accumulate, int out_dtype,
                                         const float* norm_x, const int* norm_rows, const float* gamma,
                                         const float* beta, float eps, void* k_pages, void* v_pages,
                                         const int* slots, int q_size, int kv_heads, int head_dim, int page_size,
                                         cudaStream_t stream) {
    NormArgs ln{norm_x, norm_rows, gamma, beta, eps};
    KvArgs kv{(__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, slots, q_size, kv_heads, head_dim, page_size};
    Call c{x, ldx, W, bias, out, ldo, M, N, K, act, accumulate, norm_x ? &ln : nullptr, k_pages ? &kv : nullptr, stream};
    return dispatch(c, out_dtype);
}
