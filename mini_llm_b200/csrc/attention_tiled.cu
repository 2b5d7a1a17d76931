// Causal attention of prompt portions over the paged cache on CUDA cores, tiled:
// 64 queries against 32 keys at a time, everything in 32-bit.
//
// This is the prefill attention of the true 32-bit path (float cache: no tensor core, no
// reduced-precision product) and of head sizes the tensor-core kernel does not take.  A CTA
// of 256 threads takes one tile of up to 64 consecutive new tokens of one request (the same
// tiles as the tensor-core kernel) and one head.  Key tile j covers the absolute positions
// [32j, 32j+32), whatever the cut of the prompt.  Queries sit in shared memory; a key tile is
// staged transposed ([d][key]) and a value tile as it is; a thread computes 2 x 4 scores,
// the 8 threads of a query row find the row maximum with shuffles, p = exp(s - m') goes
// through shared memory, and a thread accumulates 2 rows x head_dim/8 outputs.  The recurrence
// is the reference's (src/kernels/prefill/flashattention.cu:129-168), whose kernel reduces
// every single score over two warps with block-wide synchronisation (:7-32).
#include "common.cuh"

namespace {

constexpr int BQ = 64, BK = 32, THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_tiled_kernel(const T* q, long long q_stride, const T* k_pages,    // written by kernels of this step: no __restrict__
                       const T* v_pages, const int* __restrict__ block_table, int bt_stride,
                       const int* __restrict__ tiles, const int* __restrict__ positions, T* __restrict__ out,
                       long long out_stride, int H, int Hkv, int dh, int page_size, float scale, int window) {
    extern __shared__ float sm[];
    const int qrow = dh + 1;
    float* Qs = sm;                         // [BQ][dh+1]
    float* Kt = Qs + BQ * qrow;             // [dh][BK]
    float* Vs = Kt + dh * BK;               // [BK][dh]
    float* Ps = Vs + BK * dh;               // [BQ][BK+1]
    pdl_wait();
    pdl_launch();
    const int tile = blockIdx.y, h = blockIdx.x;                      // the host lists long tiles first
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;          // rows 2ty, 2ty+1; keys 4tx..4tx+3; dims tx + 8i
    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;

    for (int i = tid; i < BQ * dh; i += THREADS) {
        const int r = i / dh, d = i % dh;
        Qs[r * qrow + d] = r < rows ? to_f32(q[(size_t)(tok0 + r) * q_stride + (size_t)h * dh + d]) * scale : 0.f;
    }
    constexpr int MAXI = 32;                // head sizes up to 256: 32 dims per thread
    float o[2][MAXI];
#pragma unroll
    for (int i = 0; i < MAXI; ++i) { o[0][i] = 0.f; o[1][i] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int nd = dh / 8;
    const int q0 = pos0 + 2 * ty;           // absolute position of this thread's first row

    for (int j = first_key / BK; j <= pos_max / BK; ++j) {
        __syncthreads();                    // the previous tile is no longer read (and Qs is complete)
        // stage the tile.  Keys go in transposed: neighbouring threads take neighbouring keys (same piece of
        // the row), so the stores to [d][key] do not collide.  Values go in as they are: neighbouring threads
        // take neighbouring 16-byte pieces of one row.
        constexpr int VEC = 16 / sizeof(T);
        const int pieces = dh / VEC;
        for (int i = tid; i < BK * pieces; i += THREADS) {
            const int key = i % BK, piece = i / BK;
            const int kp = j * BK + key;
            float kf[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) kf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const size_t off = (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dh + piece * VEC;
                if constexpr (sizeof(T) == 4) {
                    const float4 a = *reinterpret_cast<const float4*>(k_pages + off);
                    kf[0] = a.x; kf[1] = a.y; kf[2] = a.z; kf[3] = a.w;
                } else {
                    const uint4 a = *reinterpret_cast<const uint4*>(k_pages + off);
                    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { kf[2 * e] = __low2float(a2[e]); kf[2 * e + 1] = __high2float(a2[e]); }
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) Kt[(piece * VEC + e) * BK + key] = kf[e];
        }
        for (int i = tid; i < BK * pieces; i += THREADS) {
            const int key = i / pieces, piece = i % pieces;
            const int kp = j * BK + key;
            float vf[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) vf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const size_t off = (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dh + piece * VEC;
                if constexpr (sizeof(T) == 4) {
                    const float4 b = *reinterpret_cast<const float4*>(v_pages + off);
                    vf[0] = b.x; vf[1] = b.y; vf[2] = b.z; vf[3] = b.w;
                } else {
                    const uint4 b = *reinterpret_cast<const uint4*>(v_pages + off);
                    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
                    for (int e = 0; e < 4; ++e) { vf[2 * e] = __low2float(b2[e]); vf[2 * e + 1] = __high2float(b2[e]); }
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; e += 4)
                *reinterpret_cast<float4*>(Vs + key * dh + piece * VEC + e) = make_float4(vf[e], vf[e + 1], vf[e + 2], vf[e + 3]);
        }
        __syncthreads();
        // scores: 2 rows x 4 keys per thread
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const float* qa = Qs + (2 * ty) * qrow;
        const float* qb = qa + qrow;
        for (int d = 0; d < dh; ++d) {
            const float4 kv = *reinterpret_cast<const float4*>(Kt + d * BK + 4 * tx);
            const float a = qa[d], b = qb[d];
            s[0][0] = fmaf(a, kv.x, s[0][0]); s[0][1] = fmaf(a, kv.y, s[0][1]);
            s[0][2] = fmaf(a, kv.z, s[0][2]); s[0][3] = fmaf(a, kv.w, s[0][3]);
            s[1][0] = fmaf(b, kv.x, s[1][0]); s[1][1] = fmaf(b, kv.y, s[1][1]);
            s[1][2] = fmaf(b, kv.z, s[1][2]); s[1][3] = fmaf(b, kv.w, s[1][3]);
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qp = q0 + r;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int kp = j * BK + 4 * tx + c;
                const bool vis = kp <= qp && (window <= 0 || kp > qp - window);
                s[r][c] = vis ? s[r][c] : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m_run[r], mx);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = expf(m_run[r] - muse);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = expf(s[r][c] - muse);
                Ps[(2 * ty + r) * (BK + 1) + 4 * tx + c] = p;
                rs += p;
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            l_run[r] = l_run[r] * alpha[r] + rs;
            m_run[r] = m_new;
        }
        __syncwarp();                       // a row's 8 threads are lanes of one warp: its p values are in place
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            if (i < nd) { o[0][i] *= alpha[0]; o[1][i] *= alpha[1]; }
        }
        const float* pa = Ps + (2 * ty) * (BK + 1);
        const float* pb = pa + (BK + 1);
        for (int key = 0; key < BK; ++key) {
            const float p0 = pa[key], p1 = pb[key];
            const float* vr = Vs + key * dh + tx;
#pragma unroll
            for (int i = 0; i < MAXI; ++i) {
                if (i < nd) {
                    const float v = vr[8 * i];
                    o[0][i] = fmaf(p0, v, o[0][i]);
                    o[1][i] = fmaf(p1, v, o[1][i]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = 2 * ty + r;
        if (row >= rows) continue;
        const float inv = 1.f / l_run[r];
        T* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)h * dh;
#pragma unroll
        for (int i = 0; i < MAXI; ++i)
            if (i < nd) orow[tx + 8 * i] = from_f32<T>(o[r][i] * inv);
    }
}

template <typename T>
int launch(const void* q, long long q_stride, const void* k_pages, const void* v_pages, const int* block_table,
           int bt_stride, const int* tiles, int n_tiles, const int* positions, void* out, long long out_stride, int H,
           int Hkv, int dh, int page_size, float scale, int window, cudaStream_t stream) {
    const size_t smem = ((size_t)BQ * (dh + 1) + 2 * (size_t)dh * BK + (size_t)BQ * (BK + 1)) * sizeof(float);
    auto kern = attention_tiled_kernel<T>;
    static size_t set = 0;
    if (smem > 48 * 1024 && smem > set) {
        MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = smem;
    }
    MLLM_CUDA(mllm_launch(kern, dim3(H, n_tiles), dim3(THREADS), smem, stream, true, (const T*)q, q_stride,
                          (const T*)k_pages, (const T*)v_pages, block_table, bt_stride, tiles, positions, (T*)out,
                          out_stride, H, Hkv, dh, page_size, scale, window));
    return 0;
}

}  // namespace

// tiles: n_tiles x (request index in the batch, flat index of the tile's first token, rows <= 64).
// float32 or bfloat16 cache and queries; head sizes that are multiples of 16 up to 256.
MLLM_EXPORT int mllm_attention_tiled(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                     const int* block_table, int bt_stride, const int* tiles, int n_tiles,
                                     const int* positions, void* out, long long out_stride, int H, int Hkv, int dh,
                                     int page_size, float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (dh <= 0 || dh % 16 != 0 || dh > 256)
        return mllm_fail(1, "attention_tiled: head size %d is not a multiple of 16 in 16..256", dh);
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_tiled: %d heads over %d key/value heads", H, Hkv);
    if (n_tiles > 65535) return mllm_fail(1, "attention_tiled: %d query tiles are more than one launch takes", n_tiles);
    if (dtype == MLLM_F32)
        return launch<float>(q, q_stride, k_pages, v_pages, block_table, bt_stride, tiles, n_tiles, positions, out,
                             out_stride, H, Hkv, dh, page_size, scale, window, stream);
    if (dtype == MLLM_BF16)
        return launch<__nv_bfloat16>(q, q_stride, k_pages, v_pages, block_table, bt_stride, tiles, n_tiles, positions,
                                     out, out_stride, H, Hkv, dh, page_size, scale, window, stream);
    return mllm_fail(1, "attention_tiled: unknown dtype code %d", dtype);
}
