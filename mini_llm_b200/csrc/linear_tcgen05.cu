// out = act(A[M,K] . W[N,K]^T + bias) (+ out) on the fifth-generation tensor cores:
// the product of prefill steps (many rows), bfloat16 operands, 32-bit accumulation.
//
// CTAs are persistent (one per SM) and walk over 128 x BN tiles of the result; BN is one of
// 64, 96, 128, 192, 256, chosen per shape.  Warp 0 (one elected lane) is the
// producer: it moves 128 x 64 tiles of A and BN x 64 tiles of W from global memory to a
// ring of shared-memory stages with TMA (cp.async.bulk.tensor, 128-byte swizzle; rows
// and columns beyond the matrices are filled with zeros by the copy engine, so any M, N
// and any K that is a multiple of 8 work).  Warp 1 (one lane) issues tcgen05.mma
// (cta_group::1, kind::f16, M=128, N=BN, K=16, four per stage) with the accumulator in
// tensor memory, and frees a stage with tcgen05.commit.  There are two accumulators, so
// the MMAs of the next tile run while warps 2..9, the epilogue, drain the last one: two
// warps share a quarter of the lanes and take 32-column chunks in turn; a warp reads its
// 32 lanes with tcgen05.ld, passes them through a
// small shared-memory staging area so that a store instruction covers 4 rows x 32
// consecutive columns, and applies bias, activation or the 32-bit residual sum on the way.
//
// The sum over K of one output element runs in the same order whatever M is (K tiles in
// sequence, no split over K), so a row's result does not depend on the batch.
// Every wait on an mbarrier is bounded: after the limit the kernel records an error code
// in a device word that the host reads, lets its copies land, frees its tensor memory
// and returns.
//
// The reference multiplies with FP32 SIMT tiles (src/kernels/gemm.cu:238-580), or cuBLAS
// SGEMM when MINI_LLM_USE_CUBLAS is set (:119-156); it has no tensor-core path.
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64;
constexpr int EPI_WARPS = 8;                  // two per quarter of the tensor-memory lanes
constexpr int THREADS = (2 + EPI_WARPS) * 32;

__device__ int g_tc_error = 0;          // first error code seen by any tcgen05 kernel

constexpr int tmem_cols(int bn) { return bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; }

template <int BN> struct Cfg {
    static constexpr int KB = BN <= 96 ? 2 : 1;                     // 64-wide k-blocks per stage: narrow tiles wait less often
    static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    static constexpr int BLOCK_BYTES = A_BYTES + B_BYTES;           // one k-block of A and of W
    static constexpr int STAGE_BYTES = KB * BLOCK_BYTES;            // a multiple of 1024 for every BN used
    static constexpr int EPI_ROW = 36;                              // floats per staged row: 32 + 4 of padding
    static constexpr int EPI_BYTES = EPI_WARPS * 32 * EPI_ROW * 4;  // every epilogue warp stages 32 rows
    static constexpr int BIAS_BYTES = EPI_WARPS * 128 * 4;          // every epilogue warp keeps the bias of its (up to 4) chunks
    static constexpr int STAGES = (227 * 1024 - EPI_BYTES - BIAS_BYTES - 2304) / STAGE_BYTES;   // 3 (BN=256, 96) ... 4 (BN=192, 64)
    static constexpr int ACC_COLS = tmem_cols(BN);                  // tensor-memory columns of one accumulator
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + BIAS_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
};

// Cache write fused into the epilogue of a Q|K|V projection: output columns [0, q_size) are the
// queries and go to `out`; the key and the value columns of row m go straight to the page slot
// slots[m] ([page][kv_head][offset][head_dim], slot = page * page_size + offset).  A block of 32
// columns lies inside one head (head_dim is a multiple of 32), so a lane stores 64 contiguous bytes.
struct KvOut {
    __nv_bfloat16* k_pages;      // null: a plain product
    __nv_bfloat16* v_pages;
    const int* slots;
    int q_size, kv_heads, head_dim, page_size;
};

// A persistent CTA: tiles t = blockIdx.x, blockIdx.x + gridDim.x, ...; tile -> (m tile, n tile)
// with n fastest.  Two accumulators in tensor memory let the epilogue of one tile run while
// the next tile's MMAs are issued.
template <int BN, typename TO>
__global__ void __launch_bounds__(THREADS, 1)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                      const __grid_constant__ CUtensorMap map_o, const float* __restrict__ bias, TO* out, long long ldo,
                      int M, int N, int K, int act, int accumulate, int vec_ok, int tma_out, int tiles_n,
                      int num_tiles, KvOut kv) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* epi = reinterpret_cast<float*>(tiles + (size_t)C::STAGES * C::STAGE_BYTES);       // 1024-byte aligned
    float* sbias = reinterpret_cast<float*>(tiles + (size_t)C::STAGES * C::STAGE_BYTES + C::EPI_BYTES);   // [EPI_WARPS][128]
    uint64_t* full = (uint64_t*)(tiles + (size_t)C::STAGES * C::STAGE_BYTES + C::EPI_BYTES + C::BIAS_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;          // [2]
    uint64_t* acc_empty = acc_full + 2;              // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* failed = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = (K + C::KB * BK - 1) / (C::KB * BK);       // stages per tile; k-blocks beyond K are zeros

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS); }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_slot, 2 * C::ACC_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // The weights are written by no kernel of the step: the W tiles of the first stages are asked for before the
    // wait on the previous kernel; their A tiles follow after it and complete the same barriers.
    int pre = 0;                                                 // stages whose W tiles are already on their way
    if (warp == 0 && lane == 0) {
        const int my_tiles = (int)blockIdx.x < num_tiles ? (num_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        pre = min(C::STAGES, my_tiles * nk);
        for (int g = 0; g < pre; ++g) {
            const int tile = blockIdx.x + (g / nk) * gridDim.x, kt = g % nk;
            const int n0 = (tile % tiles_n) * BN;
            uint8_t* a_dst = tiles + (size_t)g * C::STAGE_BYTES;
            mbar_expect_tx(&full[g], C::STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < C::KB; ++b)
                tma_load_2d(a_dst + b * C::BLOCK_BYTES + C::A_BYTES, &map_w, (kt * C::KB + b) * BK, n0, &full[g]);
        }
    }
    pdl_wait();                 // now what earlier kernels of the step wrote may be read
    pdl_launch();

    if (warp == 0) {
        if (lane == 0) {
            int g = 0;                                           // k-steps issued so far, over all tiles
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
                for (int kt = 0; kt < nk; ++kt, ++g) {
                    const int s = g % C::STAGES;
                    if (g >= C::STAGES && !mbar_wait(&empty[s], ((g / C::STAGES) - 1) & 1)) { *failed = 1; break; }
                    if (*failed) break;
                    uint8_t* a_dst = tiles + (size_t)s * C::STAGE_BYTES;
                    const bool w_sent = g < pre;
                    if (!w_sent) mbar_expect_tx(&full[s], C::STAGE_BYTES);
#pragma unroll
                    for (int b = 0; b < C::KB; ++b) {
                        tma_load_2d(a_dst + b * C::BLOCK_BYTES, &map_a, (kt * C::KB + b) * BK, m0, &full[s]);
                        if (!w_sent)
                            tma_load_2d(a_dst + b * C::BLOCK_BYTES + C::A_BYTES, &map_w, (kt * C::KB + b) * BK, n0, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int g = 0, ti = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*failed; tile += gridDim.x, ++ti) {
                const int buf = ti & 1;
                if (ti >= 2 && !mbar_wait(&acc_empty[buf], ((ti >> 1) - 1) & 1)) { *failed = 4; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * C::ACC_COLS);
                bool ok = true;
                for (int kt = 0; kt < nk; ++kt, ++g) {
                    const int s = g % C::STAGES;
                    if (!mbar_wait(&full[s], (g / C::STAGES) & 1)) { *failed = 2; ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + (size_t)s * C::STAGE_BYTES);
#pragma unroll
                    for (int b = 0; b < C::KB; ++b) {
                        const uint64_t a_desc = make_smem_desc(a_addr + b * C::BLOCK_BYTES);
                        const uint64_t b_desc = make_smem_desc(a_addr + b * C::BLOCK_BYTES + C::A_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)      // 32 bytes along K inside the swizzle atom = +2 in the address field
                            umma_f16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | b | k) != 0);
                    }
                    umma_commit(&empty[s]);                 // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[buf]);                // the accumulator is complete once all of them are done
            }
        }
    } else {
        const int q = warp & 3;                             // the quarter of the 128 TMEM lanes this warp may read
        const int half = (warp - 2) >> 2;                   // the two warps of a quarter take the 32-column chunks in turn
        float* stage = epi + (size_t)(warp - 2) * 32 * C::EPI_ROW;
        const int sub_r = lane >> 3, sub_c = (lane & 7) * 4;     // phase B: 4 rows x 8 lanes of 4 columns
        int ti = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++ti) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            const int buf = ti & 1;
            float* wb = sbias + (warp - 2) * 128;            // this warp's bias values: 32 per chunk it will take
            if (tma_out) {
                // fetched while the MMAs still run; nobody else reads or writes this warp's copy
#pragma unroll
                for (int k = 0; k < (BN / 32 + 1) / 2; ++k) {
                    const int n = n0 + (half + 2 * k) * 32 + lane;
                    wb[k * 32 + lane] = (bias && half + 2 * k < BN / 32 && n < N) ? __ldg(bias + n) : 0.f;
                }
                __syncwarp();
            }
            bool ok = mbar_wait(&acc_full[buf], (ti >> 1) & 1);
            if (!ok) *failed = 3;
            ok = __all_sync(0xffffffffu, ok && !*failed);   // tcgen05.ld is warp-wide: decide as a warp
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * C::ACC_COLS);
            // The accumulator is read 32 columns at a time; the load of the next 32 is in flight while
            // the current ones go through shared memory to global memory.
            constexpr int NC = BN / 32;
            uint32_t r[32];
            if (tma_out) {
                // the block of 32 rows x 32 columns goes out through the copy engine
                constexpr int ES = (int)sizeof(TO);
                uint8_t* sblk = reinterpret_cast<uint8_t*>(epi) + (size_t)(warp - 2) * 4096;    // 1024-byte aligned
                const int row0 = m0 + q * 32;
                int my_slot = -1;                            // this lane's row: where its keys and values go
                if constexpr (sizeof(TO) == 2) {
                    if (kv.k_pages && row0 + lane < M) my_slot = kv.slots[row0 + lane];
                }
                if (half < NC) {
                    tmem_ld32_issue(t_addr + (uint32_t)(half * 32), r);
                    tmem_ld_wait();
                }
                if (half + 2 >= NC) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                }
#pragma unroll 1
                for (int c = half; c < NC; c += 2) {
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 b4 = *reinterpret_cast<const float4*>(wb + (c >> 1) * 32 + 4 * j);   // same address in all lanes
                        v[4 * j] = __uint_as_float(r[4 * j]) + b4.x;
                        v[4 * j + 1] = __uint_as_float(r[4 * j + 1]) + b4.y;
                        v[4 * j + 2] = __uint_as_float(r[4 * j + 2]) + b4.z;
                        v[4 * j + 3] = __uint_as_float(r[4 * j + 3]) + b4.w;
                    }
                    if (c + 2 < NC) tmem_ld32_issue(t_addr + (uint32_t)((c + 2) * 32), r);   // r is free: refill it meanwhile
                    if (act == MLLM_ACT_GELU_TANH) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = ES == 2 ? gelu_tanh_fast(v[j]) : gelu_tanh_f(v[j]);
                    } else if (act == MLLM_ACT_GELU_ERF) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = gelu_erf_f(v[j]);
                    }
                    if constexpr (sizeof(TO) == 2) {
                        if (kv.k_pages && n0 + c * 32 >= kv.q_size) {
                            // key or value columns: straight from the registers to the row's page slot
                            if (my_slot >= 0 && n0 + c * 32 < N) {
                                const int cc = n0 + c * 32 - kv.q_size, kvs = kv.kv_heads * kv.head_dim;
                                const int which = cc / kvs, c2 = cc % kvs;
                                const int head = c2 / kv.head_dim, d0 = c2 % kv.head_dim;
                                __nv_bfloat16* dst = (which == 0 ? kv.k_pages : kv.v_pages) +
                                    (((size_t)(my_slot / kv.page_size) * kv.kv_heads + head) * kv.page_size +
                                     my_slot % kv.page_size) * kv.head_dim + d0;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    uint4 pk;
                                    __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                                    *reinterpret_cast<uint4*>(dst + 8 * j) = pk;
                                }
                            }
                            if (c + 2 < NC) tmem_ld_wait();
                            if (c + 2 < NC && c + 4 >= NC) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                            }
                            continue;
                        }
                    }
                    if (lane == 0) bulk_wait_read();         // the copy engine has read the last block out of the buffer
                    __syncwarp();
                    // lane = row; 16-byte pieces are swizzled the way the tensor map expects (128-byte rows:
                    // piece ^ (row & 7); 64-byte rows: piece ^ ((row >> 1) & 3)), which also spreads the banks
                    if constexpr (ES == 4) {
                        uint8_t* rowp = sblk + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) =
                                make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
                        uint8_t* rowp = sblk + lane * 64;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 pk;
                            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                            for (int i = 0; i < 4; ++i) hh[i] = __floats2bfloat162_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
                            *reinterpret_cast<uint4*>(rowp + ((j ^ ((lane >> 1) & 3)) << 4)) = pk;
                        }
                    }
                    fence_async_smem();                      // the writes above become visible to the copy engine
                    __syncwarp();
                    if (lane == 0 && row0 < M && n0 + c * 32 < N) {
                        if (accumulate) tma_reduce_add_2d(&map_o, n0 + c * 32, row0, sblk);
                        else tma_store_2d(&map_o, n0 + c * 32, row0, sblk);
                        bulk_commit();
                    }
                    if (c + 2 < NC) tmem_ld_wait();
                    if (c + 2 < NC && c + 4 >= NC) {         // this warp's last read of the accumulator has landed
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    }
                }
                continue;
            }
            if (half < NC) {
                tmem_ld32_issue(t_addr + (uint32_t)(half * 32), r);
                tmem_ld_wait();
            }
            if (half + 2 >= NC) {                            // that was this warp's only read (or it has none)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            }
#pragma unroll 1
            for (int c = half; c < NC; c += 2) {
                // Phase A: 32 columns of this warp's 32 rows, one row per lane, to shared memory
                float4* dst = reinterpret_cast<float4*>(stage + (size_t)lane * C::EPI_ROW);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                         __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                if (c + 2 < NC) tmem_ld32_issue(t_addr + (uint32_t)((c + 2) * 32), r);   // r is free: refill it meanwhile
                __syncwarp();
                // Phase B: each store instruction covers 4 rows x 32 consecutive columns
                const int n = n0 + c * 32 + sub_c;
                float bv[4] = {0.f, 0.f, 0.f, 0.f};
                if (bias) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) bv[i] = n + i < N ? __ldg(bias + n + i) : 0.f;
                }
                const bool vec = vec_ok && n + 4 <= N;
                // the old values of a residual sum are fetched together, ahead of the arithmetic
                float4 old[8];
                if constexpr (sizeof(TO) == 4) {
                    if (accumulate && vec) {
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int row = m0 + q * 32 + it * 4 + sub_r;
                            old[it] = (row < M && n < N) ? *reinterpret_cast<const float4*>(out + (size_t)row * ldo + n)
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                }
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + sub_r;
                    const int row = m0 + q * 32 + rr;
                    if (row >= M || n >= N) continue;
                    const float4 a = *reinterpret_cast<const float4*>(stage + (size_t)rr * C::EPI_ROW + sub_c);
                    float v[4] = {a.x + bv[0], a.y + bv[1], a.z + bv[2], a.w + bv[3]};
                    if (act == MLLM_ACT_GELU_TANH) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[i] = sizeof(TO) == 2 ? gelu_tanh_fast(v[i]) : gelu_tanh_f(v[i]);
                    } else if (act == MLLM_ACT_GELU_ERF) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[i] = gelu_erf_f(v[i]);
                    }
                    TO* o = out + (size_t)row * ldo + n;
                    if (vec) {
                        if constexpr (sizeof(TO) == 4) {
                            if (accumulate) { v[0] += old[it].x; v[1] += old[it].y; v[2] += old[it].z; v[3] += old[it].w; }
                            *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
                        } else {
                            uint2* po = reinterpret_cast<uint2*>(o);
                            if (accumulate) {
                                const uint2 ob = *po;
                                const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&ob);
                                v[0] += __low2float(oh[0]); v[1] += __high2float(oh[0]);
                                v[2] += __low2float(oh[1]); v[3] += __high2float(oh[1]);
                            }
                            uint2 pk;
                            __nv_bfloat162* hh = reinterpret_cast<__nv_bfloat162*>(&pk);
                            hh[0] = __floats2bfloat162_rn(v[0], v[1]);
                            hh[1] = __floats2bfloat162_rn(v[2], v[3]);
                            *po = pk;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (n + i < N) {
                                float x = v[i];
                                if (accumulate) x += to_f32(o[i]);
                                o[i] = from_f32<TO>(x);
                            }
                        }
                    }
                }
                if (c + 2 < NC) tmem_ld_wait();
                if (c + 2 < NC && c + 4 >= NC) {             // this warp's last read of the accumulator has landed
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                } else {
                    __syncwarp();                            // the staging rows are free for the next 32 columns
                }
            }
        }
    }
    if (warp >= 2 && lane == 0 && tma_out) bulk_wait_all();     // this thread's stores have been written
    tc_fence_before();
    __syncthreads();
    if (*failed) {
        if (threadIdx.x == 0) { atomicCAS(&g_tc_error, 0, *failed); report_to_host(100 + *failed); }
        // copies already issued may still be writing this CTA's shared memory: let them land
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * C::ACC_COLS);
    }
}

int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, typename TO>
int launch(const void* A, long long lda, const void* W, const float* bias, void* out, long long ldo, int M, int N,
           int K, int act, int accumulate, cudaStream_t stream, const KvOut& kv) {
    using C = Cfg<BN>;
    static_assert(C::STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of swizzled tiles");
    CUtensorMap ma, mw, mo;
    int rc = get_map(A, lda, M, K, BK, BM, MAP_BF16_SW128, &ma);
    if (rc) return rc;
    rc = get_map(W, K, N, K, BK, BN, MAP_BF16_SW128, &mw);
    if (rc) return rc;
    // The copy engine writes the result when its rows are 16-byte aligned; a residual sum goes through
    // it only in 32-bit (its bfloat16 addition would round the new term before adding).
    const int tma_out = (uintptr_t)out % 16 == 0 && (ldo * (long long)sizeof(TO)) % 16 == 0 &&
                        !(accumulate && sizeof(TO) == 2);
    if (kv.k_pages && !tma_out) return mllm_fail(1, "linear_tcgen05: the cache-writing epilogue needs 16-byte aligned query rows");
    if (tma_out) {
        // with the cache write fused in, `out` holds the query columns only: the map ends there
        rc = get_map(out, ldo, M, kv.k_pages ? kv.q_size : N, 32, 32, sizeof(TO) == 4 ? MAP_F32_SW128 : MAP_BF16_SW64, &mo);
        if (rc) return rc;
    } else {
        mo = ma;                                       // not used by the kernel
    }
    auto kern = linear_tcgen05_kernel<BN, TO>;
    static bool set = false;
    if (!set) {
        MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM));
        set = true;
    }
    // 4 consecutive outputs per store: 16 bytes (32-bit) or 8 bytes (bfloat16); column offsets are multiples of 4
    const int vec_ok = ((uintptr_t)out % (4 * sizeof(TO)) == 0) && (ldo % 4 == 0);
    const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM;
    const int num_tiles = tiles_n * tiles_m;
    const int grid = num_tiles < sm_count() ? num_tiles : sm_count();
    MLLM_CUDA(mllm_launch(kern, dim3(grid), dim3(THREADS), C::SMEM, stream, true, ma, mw, mo, bias, (TO*)out, ldo, M, N,
                          K, act, accumulate, vec_ok, tma_out, tiles_n, num_tiles, kv));
    return 0;
}

template <typename TO>
int pick_bn(const void* A, long long lda, const void* W, const float* bias, void* out, long long ldo, int M, int N,
            int K, int act, int accumulate, cudaStream_t stream, const KvOut& kv = KvOut{}) {
    // The tile width that moves the fewest bytes per SM: a CTA runs ceil(tiles / SMs) tiles one after
    // the other and every k-step of a tile brings in (128 + BN) rows of 64 values.
    const int widths[5] = {256, 192, 128, 96, 64};
    const long long tiles_m = (M + BM - 1) / BM;
    long long best_cost = -1;
    int best = 64;
    for (int i = 0; i < 5; ++i) {
        const int bn = widths[i];
        if (bn > 64 && bn >= 2 * N) continue;                       // far wider than the matrix
        const long long tiles = tiles_m * ((N + bn - 1) / bn);
        const long long rounds = (tiles + sm_count() - 1) / sm_count();
        const long long cost = rounds * (BM + bn) + rounds * 24;  // + a fixed part per tile (epilogue tail)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
#define GO(B) return launch<B, TO>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, stream, kv)
    switch (best) {
        case 256: GO(256);
        case 192: GO(192);
        case 128: GO(128);
        case 96: GO(96);
        default: GO(64);
    }
#undef GO
}

}  // namespace

// The pinned host word that this file's kernels write when they give up on a wait.
MLLM_EXPORT int mllm_tcgen05_bind_error(int* word) { return bind_host_error(word); }

namespace {
__global__ void report_error_kernel(int code) { report_to_host(code); }
}  // namespace

// Writes `code` to the host word from the device, the way a kernel that gave up would: lets a test check
// that the host notices, without making any wait run out.
MLLM_EXPORT int mllm_debug_report_error(int code, cudaStream_t stream) {
    report_error_kernel<<<1, 1, 0, stream>>>(code);
    MLLM_CHECK_LAUNCH("report_error_kernel");
    return 0;
}

// The first error recorded by a tcgen05 kernel since the last call (0 = none); resets it.
MLLM_EXPORT int mllm_tcgen05_error(int* code) {
    int zero = 0;
    MLLM_CUDA(cudaMemcpyFromSymbol(code, g_tc_error, sizeof(int)));
    if (*code) MLLM_CUDA(cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)));
    return 0;
}

// bfloat16 A [M,K] (row stride lda) and W [N,K]; out bfloat16 or 32-bit.  Needs K and
// lda multiples of 8 and 16-byte aligned operands (TMA's rules).
MLLM_EXPORT int mllm_linear_tcgen05(const void* A, long long lda, const void* W, const float* bias, void* out,
                                    long long ldo, int M, int N, int K, int act, int accumulate, int out_dtype,
                                    cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0)
        return mllm_fail(1, "linear_tcgen05: K=%d and the row stride %lld must be multiples of 8", K, lda);
    if ((uintptr_t)A % 16 != 0 || (uintptr_t)W % 16 != 0)
        return mllm_fail(1, "linear_tcgen05: operands must be 16-byte aligned");
    if ((M + BM - 1) / BM > 65535) return mllm_fail(1, "linear_tcgen05: M=%d exceeds the grid limit", M);
    if (out_dtype == MLLM_BF16)
        return pick_bn<__nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    if (out_dtype == MLLM_F32)
        return pick_bn<float>(A, lda, W, bias, out, ldo, M, N, K, act, accumulate, stream);
    return mllm_fail(1, "linear_tcgen05: unknown dtype code %d", out_dtype);
}

// The Q|K|V projection of many rows with the cache write fused in: out [M, q_size] (row stride ldo)
// receives the query columns, keys and values go to their page slots (slots[m] = page * page_size +
// offset, negative: not stored).  bfloat16 throughout; q_size and head_dim multiples of 32.
MLLM_EXPORT int mllm_linear_tcgen05_qkv(const void* A, long long lda, const void* W, const float* bias, void* out,
                                        long long ldo, int M, int N, int K, void* k_pages, void* v_pages,
                                        const int* slots, int q_size, int kv_heads, int head_dim, int page_size,
                                        cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0)
        return mllm_fail(1, "linear_tcgen05: K=%d and the row stride %lld must be multiples of 8", K, lda);
    if ((uintptr_t)A % 16 != 0 || (uintptr_t)W % 16 != 0) return mllm_fail(1, "linear_tcgen05: operands must be 16-byte aligned");
    if (q_size <= 0 || q_size % 32 || head_dim <= 0 || head_dim % 32 || kv_heads <= 0 || page_size <= 0 ||
        N != q_size + 2 * kv_heads * head_dim)
        return mllm_fail(1, "linear_tcgen05: %d output columns do not split into %d query and 2 x %d x %d cache columns "
                            "in blocks of 32", N, q_size, kv_heads, head_dim);
    if ((uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16) return mllm_fail(1, "linear_tcgen05: the pages must be 16-byte aligned");
    KvOut kv{(__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, slots, q_size, kv_heads, head_dim, page_size};
    return pick_bn<__nv_bfloat16>(A, lda, W, bias, out, ldo, M, N, K, MLLM_ACT_NONE, 0, stream, kv);
}
