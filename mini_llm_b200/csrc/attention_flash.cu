// Causal attention of prompt portions over the paged cache on tensor cores:
// tiles of 64 queries against tiles of 64 keys, online softmax in 32-bit registers.
//
// A CTA takes one tile of up to 64 consecutive new tokens of one request (the host cuts
// every request's portion into such tiles) and one head.  It has two groups of 4 warps (16
// query rows per warp): group 0 walks the even key tiles, group 1 the odd ones, each with
// its own online-softmax state, and the two states are merged (even, then odd) at the
// end, which halves the walk of the longest rows.  Keys and values come from the
// request's pages: tile j always covers the absolute positions [64j, 64j+64) and belongs
// to group j mod 2, so the order of the additions for a query does not depend on how the
// prompt was cut or what else is in the batch.  The host lists heavy tiles (late positions)
// first; heads are the fast grid dimension.  The two groups run on barriers of their own.
// K and V tiles are brought in with cp.async (16-byte pieces, two stages; the page numbers
// of a tile are fetched one round before its loads are issued, so no warp waits on the
// block table), S = Q.K^T and O += P.V run on
// mma.sync.m16n8k16 (bf16 in, 32-bit accumulate); the recurrence
// m' = max(m, s), alpha = exp(m - m'), p = exp(s - m'), o = o*alpha + p*v, l = l*alpha + p
// and the final o/l are the reference's (src/kernels/prefill/flashattention.cu:129-168),
// whose kernel handles one score at a time with block-wide reductions (:7-32) and reads
// the step's own QKV buffer rather than the cache (src/model/gpt2_model.cu:307-324).
// The 32-bit p enters the P.V product as two bfloat16 terms, p = hi + lo (hi = p rounded,
// lo = the rounded remainder), with one MMA each, so the softmax weights keep about 16
// bits; l sums the unrounded values.
#include "common.cuh"

namespace {

constexpr int BQ = 64, BKV = 64, WARPS = 4, GROUPS = 2;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;                     // 0 source bytes: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void group_barrier(int group) {         // the 4 warps of one group
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(WARPS * 32) : "memory");
}
// 2^x for x <= 0 (and -inf): one MUFU instruction; results below 2^-126 are flushed to zero, which a
// softmax weight that small may be.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int DH>
__global__ void __launch_bounds__(GROUPS * WARPS * 32, DH <= 64 ? 2 : 1)
attention_flash_kernel(const __nv_bfloat16* q, long long q_stride,          // q and the pages are written by kernels of this step:
                       const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages,   // no __restrict__, never the non-coherent load path
                       const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tiles,
                       const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, long long out_stride,
                       int H, int Hkv, int page_size, float scale, int window) {
    constexpr int ROW = DH + 8;                       // padded row (elements): ldmatrix rows hit distinct banks
    constexpr int CH = DH / 8;                        // 16-byte pieces per row
    extern __shared__ __align__(16) uint8_t smem[];
    const int group = threadIdx.x / (WARPS * 32), gtid = threadIdx.x % (WARPS * 32);
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
    __nv_bfloat16* sK = sQ + BQ * ROW + group * (4 * BKV * ROW);      // this group's [2][BKV][ROW]
    __nv_bfloat16* sV = sK + 2 * BKV * ROW;                           // and its [2][BKV][ROW]

    const int tile = blockIdx.y, h = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0];
    const int pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int warp = gtid >> 5, lane = gtid & 31;                   // warp inside its group
    const int g = lane >> 2, t = lane & 3;

    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;
    const int j_first = first_key / BKV, j_hi = pos_max / BKV;
    // this group's tiles: j = j_lo, j_lo + 2, ... with j mod 2 == group
    const int j_lo = j_first + ((j_first & 1) != group ? 1 : 0);

    // Q tile -> shared memory (rows beyond the tile are zeros)
    for (int i = threadIdx.x; i < BQ * CH; i += GROUPS * WARPS * 32) {
        const int r = i / CH, c = i % CH;
        cp_async16(sQ + r * ROW + c * 8, q + (size_t)(tok0 + (r < rows ? r : 0)) * q_stride + (size_t)h * DH + c * 8,
                   r < rows);
    }
    cp_commit();
    // a thread moves the same pieces of every tile: piece i = gtid + it * 128 of BKV * CH
    constexpr int ITER = (BKV * CH + WARPS * 32 - 1) / (WARPS * 32);
    int pg[ITER];                                        // page of each piece's key, -1: not visible to any row
    auto fetch_pages = [&](int j) {
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            const int i = gtid + it * WARPS * 32;
            const int kp = j * BKV + i / CH;
            const bool ok = i < BKV * CH && j <= j_hi && kp <= pos_max && kp >= first_key;
            pg[it] = ok ? bt[kp / page_size] : -1;
        }
    };
    auto load_kv = [&](int j, int stage) {               // with the pages that fetch_pages(j) brought
        __nv_bfloat16* dK = sK + stage * BKV * ROW;
        __nv_bfloat16* dV = sV + stage * BKV * ROW;
#pragma unroll
        for (int it = 0; it < ITER; ++it) {
            const int i = gtid + it * WARPS * 32;
            if (i >= BKV * CH) break;
            const int r = i / CH, c = i % CH;
            const int kp = j * BKV + r;
            const bool ok = pg[it] >= 0;
            const size_t off = ok ? (((size_t)pg[it] * Hkv + hk) * page_size + kp % page_size) * DH + c * 8 : 0;
            cp_async16(dK + r * ROW + c * 8, k_pages + off, ok);
            cp_async16(dV + r * ROW + c * 8, v_pages + off, ok);
        }
    };
    fetch_pages(j_lo);
    if (j_lo <= j_hi) load_kv(j_lo, 0);
    cp_commit();
    fetch_pages(j_lo + 2);

    float o[DH / 8][4];
#pragma unroll
    for (int i = 0; i < DH / 8; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) o[i][k] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = scale * LOG2E;
    uint32_t qa[DH / 16][4];
    const int qrow0 = pos0 + warp * 16 + g;           // absolute position of this thread's first row; second is +8
    cp_wait<1>();                                      // the queries are in (the first key tile may still fly)
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks)
        ldsm_x4(qa[ks], sQ + (warp * 16 + (lane & 15)) * ROW + ks * 16 + (lane >> 4) * 8);

    int stage = 0;
    for (int j = j_lo; j <= j_hi; j += 2, stage ^= 1) {
        if (j + 2 <= j_hi) load_kv(j + 2, stage ^ 1);
        cp_commit();
        fetch_pages(j + 4);                                // used by the next round's loads
        cp_wait<1>();
        group_barrier(group);
        const __nv_bfloat16* tK = sK + stage * BKV * ROW;
        const __nv_bfloat16* tV = sV + stage * BKV * ROW;
        // S = Q K^T : 16 rows x 64 keys per warp
        float s[BKV / 8][4];
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt)
#pragma unroll
            for (int k = 0; k < 4; ++k) s[nt][k] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DH / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < BKV / 16; ++np) {
                uint32_t b[4];
                ldsm_x4(b, tK + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * ROW + ks * 16 + ((lane >> 3) & 1) * 8);
                mma16816(s[2 * np], qa[ks], b[0], b[1]);
                mma16816(s[2 * np + 1], qa[ks], b[2], b[3]);
            }
        }
        // mask and online softmax (two rows per thread: g and g+8).  The scores stay unscaled; the scale
        // (times log2 e, positive) enters with the subtraction of the maximum as one multiply-add.
        const int kbase = j * BKV + 2 * t;
        const bool need_mask = (j * BKV + BKV - 1 > pos0 + warp * 16) || (window > 0);
        float mx[2] = {-INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
            for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int kp = kbase + nt * 8 + (k & 1);
                    const int qp = qrow0 + (k >> 1) * 8;
                    const bool vis = kp <= qp && (window <= 0 || kp > qp - window);
                    s[nt][k] = vis ? s[nt][k] : -INFINITY;
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
            mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
        }
        float alpha[2], mneg[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r] * sl2);      // running maximum of the scaled scores
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = fast_exp2(m_run[r] - muse);              // 2^(-inf) = 0 while nothing was seen
            m_run[r] = m_new;
            mneg[r] = -muse;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pa[BKV / 16][4], pb[BKV / 16][4];
#pragma unroll
        for (int nt = 0; nt < BKV / 8; ++nt) {
            const float p0 = fast_exp2(fmaf(s[nt][0], sl2, mneg[0])), p1 = fast_exp2(fmaf(s[nt][1], sl2, mneg[0]));
            const float p2 = fast_exp2(fmaf(s[nt][2], sl2, mneg[1])), p3 = fast_exp2(fmaf(s[nt][3], sl2, mneg[1]));
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            const uint32_t h01 = pack_bf16(p0, p1), h23 = pack_bf16(p2, p3);
            pa[nt >> 1][(nt & 1) * 2] = h01;
            pa[nt >> 1][(nt & 1) * 2 + 1] = h23;
            // remainders: a bfloat16 is the upper half of a float
            pb[nt >> 1][(nt & 1) * 2] = pack_bf16(p0 - __uint_as_float(h01 << 16), p1 - __uint_as_float(h01 & 0xffff0000u));
            pb[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2 - __uint_as_float(h23 << 16), p3 - __uint_as_float(h23 & 0xffff0000u));
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * alpha[r] + rs[r];
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {     // the maximum moved for some row of the warp
#pragma unroll
            for (int i = 0; i < DH / 8; ++i) {
                o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
                o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
            }
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            // all value fragments of these 16 keys first, then the hi products of every output tile, then the lo
            // ones: consecutive MMAs never wait on each other's accumulator
            uint32_t b[DH / 16][4];
#pragma unroll
            for (int dp = 0; dp < DH / 16; ++dp)
                ldsm_x4_trans(b[dp], tV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ROW + dp * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int dp = 0; dp < DH / 16; ++dp) {
                mma16816(o[2 * dp], pa[kk], b[dp][0], b[dp][1]);
                mma16816(o[2 * dp + 1], pa[kk], b[dp][2], b[dp][3]);
            }
#pragma unroll
            for (int dp = 0; dp < DH / 16; ++dp) {
                mma16816(o[2 * dp], pb[kk], b[dp][0], b[dp][1]);
                mma16816(o[2 * dp + 1], pb[kk], b[dp][2], b[dp][3]);
            }
        }
        group_barrier(group);                              // the stage may be overwritten by the next load
    }
    cp_wait<0>();
    // merge the two groups' states: the odd-tile group hands (m, l, o) over through shared memory
    float* xch = reinterpret_cast<float*>(smem) + (size_t)(warp * 32 + lane) * (DH / 2 + 4);   // the K/V stages are free
    __syncthreads();
    if (group == 1) {
        xch[0] = m_run[0]; xch[1] = m_run[1]; xch[2] = l_run[0]; xch[3] = l_run[1];
#pragma unroll
        for (int i = 0; i < DH / 8; ++i)
#pragma unroll
            for (int k = 0; k < 4; ++k) xch[4 + i * 4 + k] = o[i][k];
    }
    __syncthreads();
    if (group == 1) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float m1 = xch[r], l1 = xch[2 + r];
        const float mm = fmaxf(m_run[r], m1);
        const float muse2 = mm == -INFINITY ? 0.f : mm;
        const float a0 = fast_exp2(m_run[r] - muse2), a1 = fast_exp2(m1 - muse2);
        l_run[r] = l_run[r] * a0 + l1 * a1;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            o[i][2 * r] = o[i][2 * r] * a0 + xch[4 + i * 4 + 2 * r] * a1;
            o[i][2 * r + 1] = o[i][2 * r + 1] * a0 + xch[4 + i * 4 + 2 * r + 1] * a1;
        }
    }
    // write O / l
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + g + r * 8;
        if (row >= rows) continue;
        const float inv = 1.f / l_run[r];
        __nv_bfloat16* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)h * DH;
#pragma unroll
        for (int i = 0; i < DH / 8; ++i) {
            const uint32_t v = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
            *reinterpret_cast<uint32_t*>(orow + i * 8 + 2 * t) = v;
        }
    }
}

template <int DH>
int launch(const void* q, long long q_stride, const void* k_pages, const void* v_pages, const int* block_table,
           int bt_stride, const int* tiles, int n_tiles, const int* positions, void* out, long long out_stride,
           int H, int Hkv, int page_size, float scale, int window, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(BQ + GROUPS * 4 * BKV) * (DH + 8) * sizeof(__nv_bfloat16);
    auto kern = attention_flash_kernel<DH>;
    static bool set = false;
    if (!set && smem > 48 * 1024) {
        MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    using bf = __nv_bfloat16;
    MLLM_CUDA(mllm_launch(kern, dim3(H, n_tiles), dim3(GROUPS * WARPS * 32), smem, stream, true, (const bf*)q, q_stride,
                          (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride, tiles, positions, (bf*)out,
                          out_stride, H, Hkv, page_size, scale, window));
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_attention_flash_tile() { return BQ; }

// tiles: n_tiles x (request index in the batch, flat index of the tile's first token, rows <= 64).
// bfloat16 only; head sizes 16, 32, 64, 128.
MLLM_EXPORT int mllm_attention_flash(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                     const int* block_table, int bt_stride, const int* tiles, int n_tiles,
                                     const int* positions, void* out, long long out_stride, int H, int Hkv, int dh,
                                     int page_size, float scale, int window, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_flash: %d heads over %d key/value heads", H, Hkv);
    if (n_tiles > 65535) return mllm_fail(1, "attention_flash: %d query tiles are more than one launch takes", n_tiles);
    if (!(scale > 0.f)) return mllm_fail(1, "attention_flash: the score scale must be positive, got %g", (double)scale);
    if (q_stride % 8 || (uintptr_t)q % 16 || out_stride % 2 || (uintptr_t)out % 4)
        return mllm_fail(1, "attention_flash: queries must be 16-byte aligned, outputs 4-byte aligned");
#define GO(D) return launch<D>(q, q_stride, k_pages, v_pages, block_table, bt_stride, tiles, n_tiles, positions, out, \
                               out_stride, H, Hkv, page_size, scale, window, stream)
    switch (dh) {
        case 16: GO(16);
        case 32: GO(32);
        case 64: GO(64);
        case 128: GO(128);
    }
#undef GO
    return mllm_fail(1, "attention_flash: head size %d is not one of 16, 32, 64, 128", dh);
}
