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

// ---------------------------------------------------------------------------------------------------------
// The same attention for long prompt portions with heads up to 64: 128 queries against 128 keys at a time, both
// products with 8 x 8 outputs per thread, the arithmetic-to-shared-memory ratio of a tiled SGEMM (64 fused
// multiply-adds per four 16-byte reads).  Key tile j covers the absolute positions [128j, 128j + 128).
//
// Scores: thread (tr, tk) of 16 x 16 takes the queries 8tr .. 8tr+7 and the keys 8tk .. 8tk+7; queries and keys lie
// in shared memory d-major ([d][row], [d][key]), so a step of d reads two float4 of each.  The 16 threads of a query
// row are the lanes of half a warp: row maxima and sums take four shuffles.  p = exp(s - m') goes to shared memory
// key-major ([key][query]).  Outputs: the two halves of the CTA take the even and the odd 64 keys of the tile, and
// within a half thread (tr, td) of 16 x 8 takes the queries 8tr .. 8tr+7 and the dims 8td .. 8td+7 (DT = head
// size / 8 dims per thread); the halves' sums meet once, at the very end, lower half first.
constexpr int WQ = 128, WK = 128;
constexpr int PW = WQ + 4;               // floats per key row of p: neighbouring keys fall on different banks

template <typename T, int DT>
__global__ void __launch_bounds__(THREADS, 1)
attention_tiled_wide_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tiles,
                            const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int H, int Hkv,
                            int page_size, float scale, int window) {
    constexpr int DH = 8 * DT;
    extern __shared__ __align__(16) float sm[];
    float* Qt = sm;                          // [DH][WQ]  queries, d-major, scaled
    float* Kt = Qt + DH * WQ;                // [DH][WK]  keys, d-major
    float* Vs = Kt + DH * WK;                // [WK][DH]  values as they are
    float* Pt = Vs + WK * DH;                // [WK][PW]  p, key-major; at the end the upper half's outputs
    float* As = Pt + WK * PW;                // [WQ] alpha of the tile, then 1 / l
    pdl_wait();
    pdl_launch();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x;
    const int tr = tid >> 4, tk = tid & 15;                  // scores: queries 8tr.., keys 8tk..
    const int half = tid >> 7, pr = (tid & 127) >> 3, td = tid & 7;   // outputs: keys of parity `half`, queries 8pr.., dims 8td.. (DT each)
    int first_key = 0;
    if (window > 0 && pos0 - window + 1 > 0) first_key = pos0 - window + 1;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int PIECES = DH / VEC;

    for (int i = tid; i < WQ * PIECES; i += THREADS) {       // neighbouring threads take neighbouring queries
        const int r = i % WQ, piece = i / WQ;
        float qf[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) qf[e] = 0.f;
        if (r < rows) {
            const T* src = q + (size_t)(tok0 + r) * q_stride + (size_t)h * DH + piece * VEC;
            if constexpr (sizeof(T) == 4) {
                const float4 a = *reinterpret_cast<const float4*>(src);
                qf[0] = a.x; qf[1] = a.y; qf[2] = a.z; qf[3] = a.w;
            } else {
                const uint4 a = *reinterpret_cast<const uint4*>(src);
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
                for (int e = 0; e < 4; ++e) { qf[2 * e] = __low2float(a2[e]); qf[2 * e + 1] = __high2float(a2[e]); }
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) Qt[(piece * VEC + e) * WQ + r] = qf[e] * scale;
    }
    float o[8][DT];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int d = 0; d < DT; ++d) o[i][d] = 0.f;
    float m_run[8], l_run[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { m_run[i] = -INFINITY; l_run[i] = 0.f; }

    for (int j = first_key / WK; j <= pos_max / WK; ++j) {
        __syncthreads();                    // the previous tile is no longer read (and Qt is complete)
        for (int i = tid; i < WK * PIECES; i += THREADS) {   // keys d-major: neighbouring threads, neighbouring keys
            const int key = i % WK, piece = i / WK;
            const int kp = j * WK + key;
            float kf[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) kf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const size_t off = (((size_t)page * Hkv + hk) * page_size + kp % page_size) * DH + piece * VEC;
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
            for (int e = 0; e < VEC; ++e) Kt[(piece * VEC + e) * WK + key] = kf[e];
        }
        for (int i = tid; i < WK * PIECES; i += THREADS) {   // values as they are: neighbouring threads, neighbouring pieces
            const int key = i / PIECES, piece = i % PIECES;
            const int kp = j * WK + key;
            float vf[VEC];
#pragma unroll
            for (int e = 0; e < VEC; ++e) vf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const size_t off = (((size_t)page * Hkv + hk) * page_size + kp % page_size) * DH + piece * VEC;
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
                *reinterpret_cast<float4*>(Vs + key * DH + piece * VEC + e) = make_float4(vf[e], vf[e + 1], vf[e + 2], vf[e + 3]);
        }
        __syncthreads();
        // scores: 8 queries x 8 keys per thread
        float s[8][8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int c = 0; c < 8; ++c) s[i][c] = 0.f;
#pragma unroll 4
        for (int d = 0; d < DH; ++d) {
            const float4 qa = *reinterpret_cast<const float4*>(Qt + d * WQ + 8 * tr);
            const float4 qb = *reinterpret_cast<const float4*>(Qt + d * WQ + 8 * tr + 4);
            const float4 ka = *reinterpret_cast<const float4*>(Kt + d * WK + 8 * tk);
            const float4 kb = *reinterpret_cast<const float4*>(Kt + d * WK + 8 * tk + 4);
            const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int c = 0; c < 8; ++c) s[i][c] = fmaf(qv[i], kv[c], s[i][c]);
        }
        const bool diagonal = j * WK + WK - 1 > pos0 || window > 0 || j * WK < first_key;   // some score of the tile may be hidden
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int qp = pos0 + 8 * tr + i;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (diagonal) {
                    const int kp = j * WK + 8 * tk + c;
                    const bool vis = kp <= qp && kp >= first_key && (window <= 0 || kp > qp - window);
                    s[i][c] = vis ? s[i][c] : -INFINITY;
                }
                mx = fmaxf(mx, s[i][c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            const float m_new = fmaxf(m_run[i], mx);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = expf(m_run[i] - muse);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                s[i][c] = expf(s[i][c] - muse);
                rs += s[i][c];
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            rs += __shfl_xor_sync(0xffffffffu, rs, 8);
            l_run[i] = l_run[i] * alpha + rs;
            m_run[i] = m_new;
            if (tk == 0) As[8 * tr + i] = alpha;
        }
        // p, key-major: a key's 8 queries of this thread are two float4
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float* dst = Pt + (8 * tk + c) * PW + 8 * tr;
            *reinterpret_cast<float4*>(dst) = make_float4(s[0][c], s[1][c], s[2][c], s[3][c]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(s[4][c], s[5][c], s[6][c], s[7][c]);
        }
        __syncthreads();
        // outputs: 8 queries x DT dims per thread over the keys of this half's parity
        {
            const float4 a0 = *reinterpret_cast<const float4*>(As + 8 * pr);
            const float4 a1 = *reinterpret_cast<const float4*>(As + 8 * pr + 4);
            const float al[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int d = 0; d < DT; ++d) o[i][d] *= al[i];
        }
#pragma unroll 2
        for (int key = half; key < WK; key += 2) {
            const float4 pa = *reinterpret_cast<const float4*>(Pt + key * PW + 8 * pr);
            const float4 pb = *reinterpret_cast<const float4*>(Pt + key * PW + 8 * pr + 4);
            const float pv[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
            float vv[DT];
#pragma unroll
            for (int d = 0; d < DT; d += 2) {
                const float2 v2 = *reinterpret_cast<const float2*>(Vs + key * DH + DT * td + d);
                vv[d] = v2.x;
                vv[d + 1] = v2.y;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int d = 0; d < DT; ++d) o[i][d] = fmaf(pv[i], vv[d], o[i][d]);
        }
    }
    // 1 / l per query, from the score threads; then the halves' outputs meet (lower half + upper half)
    __syncthreads();
    if (tk == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) As[8 * tr + i] = 1.f / l_run[i];
    }
    float* Ou = Pt;                          // [WQ][DH] the upper half's sums
    if (half == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int d = 0; d < DT; ++d) Ou[(8 * pr + i) * DH + DT * td + d] = o[i][d];
    }
    __syncthreads();
    if (half == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = 8 * pr + i;
            if (row >= rows) continue;
            const float inv = As[row];
            T* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)h * DH + DT * td;
#pragma unroll
            for (int d = 0; d < DT; ++d) orow[d] = from_f32<T>((o[i][d] + Ou[row * DH + DT * td + d]) * inv);
        }
    }
}

template <typename T, int DT>
int launch_wide(const void* q, long long q_stride, const void* k_pages, const void* v_pages, const int* block_table,
                int bt_stride, const int* tiles, int n_tiles, const int* positions, void* out, long long out_stride,
                int H, int Hkv, int page_size, float scale, int window, cudaStream_t stream) {
    constexpr int DH = 8 * DT;
    const size_t smem = ((size_t)DH * WQ + (size_t)DH * WK + (size_t)WK * DH + (size_t)WK * PW + WQ) * sizeof(float);
    auto kern = attention_tiled_wide_kernel<T, DT>;
    static bool set = false;
    if (!set) {
        MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set = true;
    }
    MLLM_CUDA(mllm_launch(kern, dim3(H, n_tiles), dim3(THREADS), smem, stream, true, (const T*)q, q_stride,
                          (const T*)k_pages, (const T*)v_pages, block_table, bt_stride, tiles, positions, (T*)out,
                          out_stride, H, Hkv, page_size, scale, window));
    return 0;
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

// The same with tiles of up to 128 rows (n_tiles x (request index, first token, rows <= 128)) for head sizes 16, 32, 48
// and 64: the kernel for long prompt portions.
MLLM_EXPORT int mllm_attention_tiled_wide(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                          const int* block_table, int bt_stride, const int* tiles, int n_tiles,
                                          const int* positions, void* out, long long out_stride, int H, int Hkv, int dh,
                                          int page_size, float scale, int window, int dtype, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_tiled_wide: %d heads over %d key/value heads", H, Hkv);
    if (n_tiles > 65535) return mllm_fail(1, "attention_tiled_wide: %d query tiles are more than one launch takes", n_tiles);
    if (page_size <= 0) return mllm_fail(1, "attention_tiled_wide: page size %d", page_size);
#define GO(TT, DT)                                                                                                   \
    return launch_wide<TT, DT>(q, q_stride, k_pages, v_pages, block_table, bt_stride, tiles, n_tiles, positions, out,  \
                               out_stride, H, Hkv, page_size, scale, window, stream)
    if (dtype == MLLM_F32) {
        switch (dh) {
            case 16: GO(float, 2);
            case 32: GO(float, 4);
            case 48: GO(float, 6);
            case 64: GO(float, 8);
        }
    } else if (dtype == MLLM_BF16) {
        switch (dh) {
            case 16: GO(__nv_bfloat16, 2);
            case 32: GO(__nv_bfloat16, 4);
            case 48: GO(__nv_bfloat16, 6);
            case 64: GO(__nv_bfloat16, 8);
        }
    } else {
        return mllm_fail(1, "attention_tiled_wide: unknown dtype code %d", dtype);
    }
#undef GO
    return mllm_fail(1, "attention_tiled_wide: head size %d is not 16, 32, 48 or 64", dh);
}
