// Causal attention of prompt portions over the paged cache on the fifth-generation tensor
// cores: tiles of 128 queries against blocks of 128 keys, head size 64, bfloat16.
//
// A CTA takes one tile of up to 128 consecutive new tokens of one request and one head.
// Warp 0 is the producer: the query tile and, block by block, the key and value pages come
// in through TMA (cp.async.bulk.tensor, 128-byte swizzle; a page of 8, 16 ... 128 tokens of
// one head is a box of page_size rows x 64 values; pages that no row of the tile can see
// are fetched from beyond the pool, which the copy engine fills with zeros).  Warp 1 (one
// lane) issues the MMAs: S = Q.K^T (tcgen05.mma 128 x 128 x 16, four per block) into tensor
// memory, and, once the softmax warps have turned S into weights, O_blk = P.V (128 x 64 x 16,
// eight per term; V is read as it lies in the pages, an MN-major operand) into a second range
// of tensor memory.  Warps 2-17 are the softmax: four threads share a query row (a warp may
// only read its own quarter of the tensor memory's lanes, and one warp reads it slowly, about
// 5 GB/s, so sixteen warps read side by side); each reads 32 of the block's 128 scores with
// tcgen05.ld, the four exchange their maxima through shared memory, and they keep the online
// softmax of the row in 32-bit registers
//   m' = max(m, s), alpha = exp(m - m'), p = exp(s - m'), o = o*alpha + p.v, l = l*alpha + sum p
// (the reference's recurrence, src/kernels/prefill/flashattention.cu:129-168, with base-2
// exponentials and the scale folded in), write the weights of the block to shared memory as
// two bfloat16 terms p = hi + lo (the product then keeps about 16 bits of them), and add
// O_blk into their row of o.  S and the weights are double-buffered: the MMAs of S for block
// i+1 are issued before those of P.V for block i, and a softmax thread adds O_blk of block i
// only after it has turned S of block i+1 into weights, so neither side waits for the other's
// hand-over (an mbarrier round trip costs about as much as the arithmetic of a block).
//
// Block j always covers the absolute positions [128 j, 128 j + 128), so the order of the
// additions for a query does not depend on how the prompt was cut or what else is in the
// batch.  Every wait on an mbarrier is bounded; after the limit the kernel records an
// error code that the host reads, lets its copies land, frees its tensor memory and returns.
//
// The reference's prefill attention handles one score at a time with block-wide reductions
// (src/kernels/prefill/flashattention.cu:7-32) and reads the step's own Q|K|V buffer.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BQ = 128, BKV = 128, DH = 64;
constexpr int PARTS = 4;                             // threads per query row: each takes 32 keys of a block and 16 of the 64 output values
constexpr int SOFTMAX_WARPS = 4 * PARTS;
constexpr int THREADS = (3 + SOFTMAX_WARPS) * 32;  // key producer, MMA issuer, softmax warps, value producer
constexpr int Q_BYTES = BQ * DH * 2;                 // 16 KB
constexpr int KV_BYTES = BKV * DH * 2;               // 16 KB each for K and V of a block
constexpr int P_BYTES = BQ * BKV * 2;                // 32 KB per term: two sub-tiles of 128 rows x 64 keys
constexpr int STAGES = 2;
constexpr int XCH_BYTES = 2 * PARTS * BQ * 4;        // partial row maxima, double-buffered; reused for the row sums at the end
constexpr size_t SMEM = 1024 + Q_BYTES + STAGES * 2 * KV_BYTES + 2 * 2 * P_BYTES + XCH_BYTES + 512;
constexpr uint32_t TMEM_COLS = 512;                  // S of even blocks in columns 0..127, of odd blocks in 128..255, O_blk in 256..319
constexpr uint32_t TMEM_O = 256;
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_error = 0;                     // first error code seen by this kernel

// Instruction descriptor with the B operand MN-major (bit 16): D=F32, A=B=BF16.
__host__ __device__ constexpr uint32_t make_idesc_bmn(int m, int n) { return make_idesc(m, n) | (1u << 16); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                         int bt_stride, const int* __restrict__ tiles, const int* __restrict__ positions,
                         __nv_bfloat16* __restrict__ out, long long out_stride, int H, int Hkv, int page_size,
                         int pool_rows, float scale, int window) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = base;
    uint8_t* sKV = sQ + Q_BYTES;                                  // [STAGES][K 16 KB | V 16 KB]
    uint8_t* sP = sKV + STAGES * 2 * KV_BYTES;                    // [2 buffers][hi term | lo term]
    float* xch = reinterpret_cast<float*>(sP + 2 * 2 * P_BYTES);  // [2][PARTS][BQ]
    uint64_t* q_full = (uint64_t*)(sP + 2 * 2 * P_BYTES + XCH_BYTES);
    uint64_t* k_full = q_full + 1;                                // [STAGES]
    uint64_t* k_empty = k_full + STAGES;                          // [STAGES]: keys are free again once S was computed
    uint64_t* v_full = k_empty + STAGES;                          // [STAGES]
    uint64_t* v_empty = v_full + STAGES;                          // [STAGES]: values are free again once P V was computed
    uint64_t* s_full = v_empty + STAGES;                          // [2]: one per S buffer
    uint64_t* p_full = s_full + 2;
    uint64_t* o_full = p_full + 1;
    uint64_t* o_free = o_full + 1;
    uint32_t* tmem_slot = (uint32_t*)(o_free + 1);
    volatile int* failed = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.x, tile = blockIdx.y;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
        }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(p_full, SOFTMAX_WARPS);
        mbar_init(o_full, 1);
        mbar_init(o_free, SOFTMAX_WARPS);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();
    pdl_launch();

    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0];
    const int pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;
    const int j_lo = first_key / BKV, j_hi = pos_max / BKV;
    const int nblk = j_hi - j_lo + 1;

    const int V_WARP = 2 + SOFTMAX_WARPS;
    if (warp == 0 || warp == V_WARP) {
        // ---------------------------------------------------------------- producers: warp 0 brings the queries and
        // the keys, the last warp the values, each as soon as the stage it writes to is free
        const bool keys = warp == 0;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        uint64_t* full = keys ? k_full : v_full;
        uint64_t* empty = keys ? k_empty : v_empty;
        const int ppb = BKV / page_size;                          // pages per block
        const int* bt = block_table + (size_t)seq * bt_stride;
        if (keys && lane == 0) {
            mbar_expect_tx(q_full, Q_BYTES);
            tma_load_2d(sQ, &map_q, h * DH, tok0, q_full);
        }
        for (int i = 0; i < nblk; ++i) {
            const int j = j_lo + i, s = i % STAGES;
            bool ok = true;
            if (lane == 0) {
                if (i >= STAGES) ok = mbar_wait(&empty[s], ((i / STAGES) - 1) & 1);
                if (!ok) *failed = 1;
                if (ok && !*failed) mbar_expect_tx(&full[s], KV_BYTES);
            }
            ok = __shfl_sync(0xffffffffu, (int)(ok && !*failed), 0) != 0;
            if (!ok) break;
            // lane p brings page p of the block: keys [128 j + p * page_size, + page_size)
            for (int p = lane; p < ppb; p += 32) {
                const int k0 = j * BKV + p * page_size;
                int row = pool_rows;                              // beyond the pool: the box is filled with zeros
                if (k0 <= pos_max && k0 + page_size > first_key) {
                    const int page = bt[k0 / page_size];
                    if (page >= 0) row = (page * Hkv + hk) * page_size;
                }
                uint8_t* dst = sKV + (size_t)s * 2 * KV_BYTES + (keys ? 0 : KV_BYTES) + (size_t)p * page_size * (DH * 2);
                tma_load_2d(dst, map, 0, row, &full[s]);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(BQ, BKV);
            constexpr uint32_t idesc_o = make_idesc_bmn(BQ, DH);
            const uint32_t t_o = tmem_base + TMEM_O;
            const uint64_t q_desc = make_smem_desc(smem_u32(sQ));
            auto issue_s = [&](int i) {                       // S(i) = Q K(i)^T into the S buffer i & 1
                const uint64_t k_desc = make_smem_desc(smem_u32(sKV + (size_t)(i % STAGES) * 2 * KV_BYTES));
#pragma unroll
                for (int k = 0; k < DH / 16; ++k)
                    umma_f16(tmem_base + (uint32_t)(i & 1) * 128, q_desc + 2 * k, k_desc + 2 * k, idesc_s, k != 0);
                umma_commit(&s_full[i & 1]);
                umma_commit(&k_empty[i % STAGES]);             // the keys of this block have been read
            };
            bool ok = mbar_wait(q_full, 0) && mbar_wait(&k_full[0], 0);
            if (!ok) *failed = 2;
            if (ok) {
                tc_fence_after();
                issue_s(0);
            }
            for (int i = 0; i < nblk && ok && !*failed; ++i) {
                if (i + 1 < nblk) {
                    // S of the next block goes ahead of this block's P V: its buffer was read two blocks ago
                    if (!mbar_wait(&k_full[(i + 1) % STAGES], ((i + 1) / STAGES) & 1)) { *failed = 3; break; }
                    tc_fence_after();
                    issue_s(i + 1);
                }
                // O_blk = P(i) V(i) (hi term, then lo term) once the weights are written and O_blk of block i-1 was read
                if (!mbar_wait(p_full, i & 1)) { *failed = 4; break; }
                if (i > 0 && !mbar_wait(o_free, (i - 1) & 1)) { *failed = 5; break; }
                if (!mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1)) { *failed = 6; break; }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sKV + (size_t)(i % STAGES) * 2 * KV_BYTES + KV_BYTES);
                const uint32_t p_addr = smem_u32(sP + (size_t)(i & 1) * 2 * P_BYTES);
#pragma unroll
                for (int term = 0; term < 2; ++term) {
#pragma unroll
                    for (int kk = 0; kk < BKV / 16; ++kk) {
                        const uint64_t a_desc = make_smem_desc(p_addr + term * P_BYTES + (kk / 4) * (P_BYTES / 2)) + 2 * (kk % 4);
                        const uint64_t b_desc = make_smem_desc(v_addr + kk * 2048);
                        umma_f16(t_o, a_desc, b_desc, idesc_o, (term | kk) != 0);
                    }
                }
                umma_commit(o_full);
                umma_commit(&v_empty[i % STAGES]);            // this block's values have been read
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax: one query row per thread
        const int q4 = warp & 3;                              // the quarter of the tensor-memory lanes this warp may read
        const int part = (warp - 2) >> 2;                     // which 32 keys of a block and which 16 output values
        const int r = q4 * 32 + lane;                         // row of the tile
        const int qp = pos0 + r;                              // its absolute position (rows beyond the tile are not stored)
        const uint32_t t_lane = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const uint32_t t_o = t_lane + TMEM_O + part * 16;
        const float sl2 = scale * LOG2E;
        float o[16];
#pragma unroll
        for (int d = 0; d < 16; ++d) o[d] = 0.f;
        float m_run = -INFINITY, l_part = 0.f, alpha_prev = 1.f;
        // A warp that gave up on a wait stays in step with the three that share its rows: it skips the work but
        // still arrives at their barriers, which also carry whether all of them are still running, so nobody waits for a warp that left.
        bool alive = true;
        uint32_t v[32];
        auto row_barrier = [&](bool fine) -> bool {          // barrier of the 4 warps of this quarter; true if all are fine
            uint32_t all;
            asm volatile(
                "{\n\t.reg .pred p, q;\n\t"
                "setp.ne.b32 p, %1, 0;\n\t"
                "bar.red.and.pred q, %2, %3, p;\n\t"
                "selp.u32 %0, 1, 0, q;\n\t}"
                : "=r"(all) : "r"((uint32_t)fine), "r"(1 + q4), "n"(PARTS * 32) : "memory");
            return all != 0;
        };
        // o = o * alpha + O_blk for the block whose P V was issued last
        auto add_block = [&](int i, float alpha) -> bool {
            bool fine = mbar_wait(o_full, i & 1);
            if (!fine) *failed = 8;
            fine = __all_sync(0xffffffffu, fine && !*failed);
            if (!fine) return false;
            tc_fence_after();
            uint32_t w[16];
            tmem_ld16(t_o, w);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = fmaf(o[e], alpha, __uint_as_float(w[e]));
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free);
            return true;
        };
        for (int i = 0; i < nblk; ++i) {
            const int j = j_lo + i;
            if (alive) {
                bool got = mbar_wait(&s_full[i & 1], (i >> 1) & 1);
                if (!got) *failed = 7;
                alive = __all_sync(0xffffffffu, got && !*failed);
            }
            const int k0 = j * BKV + part * 32;                   // first key of this thread's 32
            const bool need_mask = (j * BKV + BKV - 1 > pos0) || (window > 0);     // uniform over the CTA
            float sc[32];
            float mx = -INFINITY;
            if (alive) {
                tc_fence_after();
                tmem_ld32_issue(t_lane + (uint32_t)(i & 1) * 128 + part * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    float sv = __uint_as_float(v[e]);
                    if (need_mask && (k0 + e > qp || (window > 0 && k0 + e <= qp - window))) sv = -INFINITY;
                    sc[e] = sv;
                    mx = fmaxf(mx, sv);
                }
            }
            // the row's maximum over the block: the four threads of the row meet in shared memory
            float* xb = xch + (i & 1) * PARTS * BQ;
            xb[part * BQ + r] = mx;
            alive = row_barrier(alive);
            if (!alive) continue;                                 // all four warps of the quarter take this branch together
#pragma unroll
            for (int p = 0; p < PARTS; ++p) mx = fmaxf(mx, xb[p * BQ + r]);
            const float m_new = fmaxf(m_run, mx * sl2);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = fast_exp2(m_run - muse);
            m_run = m_new;
            // weights -> shared memory as hi + lo, their sum
            uint8_t* dst_hi = sP + (size_t)(i & 1) * 2 * P_BYTES + (part / 2) * (P_BYTES / 2) + (size_t)r * 128;
            uint8_t* dst_lo = dst_hi + P_BYTES;
            float rs = 0.f;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {                      // 8 keys = one 16-byte piece
                uint32_t hi4[4], lo4[4];
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2) {
                    const int e = g8 * 8 + e2 * 2;
                    const float p0 = fast_exp2(fmaf(sc[e], sl2, -muse)), p1 = fast_exp2(fmaf(sc[e + 1], sl2, -muse));
                    rs += p0 + p1;
                    const uint32_t hh = pack_bf16(p0, p1);
                    hi4[e2] = hh;
                    lo4[e2] = pack_bf16(p0 - __uint_as_float(hh << 16), p1 - __uint_as_float(hh & 0xffff0000u));
                }
                const int piece = (part & 1) * 4 + g8;            // 16-byte piece of the 128-byte row; swizzled by r & 7 as the MMA expects
                const int off = ((piece ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(dst_hi + off) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
                *reinterpret_cast<uint4*>(dst_lo + off) = make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]);
            }
            l_part = l_part * alpha + rs;
            fence_async_smem();                                   // the weights become visible to the tensor core's reads
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            // the block before this one: its P V has had the time of this block's softmax to finish
            if (i > 0) alive = add_block(i - 1, alpha_prev);
            alpha_prev = alpha;
        }
        if (alive) alive = add_block(nblk - 1, alpha_prev);
        // the row's sum: the four partial sums added in a fixed order
        alive = row_barrier(alive);                               // the last maxima have been read
        xch[part * BQ + r] = l_part;
        alive = row_barrier(alive);
        if (alive && r < rows) {
            float l = 0.f;
#pragma unroll
            for (int p = 0; p < PARTS; ++p) l += xch[p * BQ + r];
            const float inv = 1.f / l;
            __nv_bfloat16* orow = out + (size_t)(tok0 + r) * out_stride + (size_t)h * DH + part * 16;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint4 pk;
                pk.x = pack_bf16(o[c * 8] * inv, o[c * 8 + 1] * inv);
                pk.y = pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
                pk.z = pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
                pk.w = pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
                *reinterpret_cast<uint4*>(orow + c * 8) = pk;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*failed) {
        if (threadIdx.x == 0) { atomicCAS(&g_attn_error, 0, *failed); report_to_host(200 + *failed); }
        for (int i = 0; i < 2000; ++i) __nanosleep(100);          // copies already issued may still be landing
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace

MLLM_EXPORT int mllm_attention_tcgen05_tile() { return BQ; }

// The pinned host word that this file's kernels write when they give up on a wait.
MLLM_EXPORT int mllm_attention_tcgen05_bind_error(int* word) { return bind_host_error(word); }

// The first error recorded by the kernel since the last call (0 = none); resets it.
MLLM_EXPORT int mllm_attention_tcgen05_error(int* code) {
    int zero = 0;
    MLLM_CUDA(cudaMemcpyFromSymbol(code, g_attn_error, sizeof(int)));
    if (*code) MLLM_CUDA(cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int)));
    return 0;
}

// tiles: n_tiles x (request index in the batch, flat index of the tile's first token, rows <= 128).
// bfloat16, head size 64, pages of 8, 16, 32, 64 or 128 tokens; q [T, *] with row stride q_stride
// (elements), 16-byte aligned; k_pages / v_pages [num_pages, Hkv, page_size, 64] contiguous.
MLLM_EXPORT int mllm_attention_tcgen05(const void* q, long long q_stride, int T, const void* k_pages,
                                       const void* v_pages, int num_pages, const int* block_table, int bt_stride,
                                       const int* tiles, int n_tiles, const int* positions, void* out,
                                       long long out_stride, int H, int Hkv, int dh, int page_size, float scale,
                                       int window, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (dh != DH) return mllm_fail(1, "attention_tcgen05: head size %d is not 64", dh);
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_tcgen05: %d heads over %d key/value heads", H, Hkv);
    if (page_size < 8 || page_size > BKV || (page_size & (page_size - 1)))
        return mllm_fail(1, "attention_tcgen05: page size %d is not a power of two in 8..128", page_size);
    if (n_tiles > 65535) return mllm_fail(1, "attention_tcgen05: %d query tiles are more than one launch takes", n_tiles);
    if (!(scale > 0.f)) return mllm_fail(1, "attention_tcgen05: the score scale must be positive, got %g", (double)scale);
    if (q_stride % 8 || (uintptr_t)q % 16 || out_stride % 8 || (uintptr_t)out % 16)
        return mllm_fail(1, "attention_tcgen05: queries and outputs must be 16-byte aligned");
    if ((uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16)
        return mllm_fail(1, "attention_tcgen05: the page pools must be 16-byte aligned");
    const long long pool_rows = (long long)num_pages * Hkv * page_size;
    if (pool_rows + page_size > 2147483647LL) return mllm_fail(1, "attention_tcgen05: the page pool is too large");
    CUtensorMap mq, mk, mv;
    int rc = get_map(q, q_stride, T, H * DH, DH, BQ, MAP_BF16_SW128, &mq);
    if (rc) return rc;
    rc = get_map(k_pages, DH, (int)pool_rows, DH, DH, page_size, MAP_BF16_SW128, &mk);
    if (rc) return rc;
    rc = get_map(v_pages, DH, (int)pool_rows, DH, DH, page_size, MAP_BF16_SW128, &mv);
    if (rc) return rc;
    auto kern = attention_tcgen05_kernel;
    static bool set = false;
    if (!set) {
        MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        set = true;
    }
    using bf = __nv_bfloat16;
    MLLM_CUDA(mllm_launch(kern, dim3(H, n_tiles), dim3(THREADS), SMEM, stream, true, mq, mk, mv, block_table, bt_stride,
                          tiles, positions, (bf*)out, out_stride, H, Hkv, page_size, (int)pool_rows, scale, window));
    return 0;
}
