// Causal attention of a mixed batch over the paged cache, one warp per (token, head).
//
// Every token of the step (a prompt portion's token or a decoded one) carries its
// request's index in the batch and its absolute position p; it attends to the
// cached keys at positions max(0, p-window+1) .. p of its own request, found through
// the request's block table.  Scores, softmax and the weighted sum are 32-bit
// (expf, not the fast intrinsic); the softmax is the online form of the reference's
// prefill kernel (src/kernels/prefill/flashattention.cu:129-168: m' = max(m,s),
// alpha = exp(m-m'), p = exp(s-m'), o = o*alpha + p*v, l = l*alpha + p, out = o/l)
// taken 32 keys at a time, over pages like its decode kernel
// (src/kernels/decode/paged_attention.cu:60-120, without the +1e-6 of :97).
//
// Key chunks start at multiples of 32 counted from position 0, so the order of the
// additions for a token depends on its position only, not on how the step was cut
// or batched.  This kernel serves the 32-bit path and is the plain twin of the
// tensor-core attention; cache, queries and output share one dtype.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_DH = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* q, long long q_stride, const T* k_pages,     // written by kernels of this step: no __restrict__
                      const T* v_pages, const int* __restrict__ block_table, int bt_stride,
                      const int* __restrict__ token_seq, const int* __restrict__ positions, T* __restrict__ out,
                      long long out_stride, int T_tokens, int H, int Hkv, int dh, int page_size, float scale,
                      int window) {
    __shared__ float qs[WARPS][MAX_DH];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    if (gw >= (long long)T_tokens * H) return;
    const int t = (int)(gw / H), h = (int)(gw % H);
    const int hk = h / (H / Hkv);
    const int seq = token_seq[t], p = positions[t];
    const int* bt = block_table + (size_t)seq * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * dh;
    for (int d = lane; d < dh; d += 32) qs[warp][d] = to_f32(qrow[d]);
    __syncwarp();

    int first = 0;
    if (window > 0 && p - window + 1 > 0) first = p - window + 1;
    constexpr int NACC = MAX_DH / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int c0 = (first / 32) * 32; c0 <= p; c0 += 32) {
        const int kp = c0 + lane;
        const bool valid = kp >= first && kp <= p;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[kp / page_size];
            const T* kr = k_pages + (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dh;
            float dot = 0.f;
            for (int d = 0; d < dh; d += 8) {
                float kv[8];
                if constexpr (sizeof(T) == 4) {
                    const float4 a = *reinterpret_cast<const float4*>(kr + d);
                    const float4 b = *reinterpret_cast<const float4*>(kr + d + 4);
                    kv[0] = a.x; kv[1] = a.y; kv[2] = a.z; kv[3] = a.w;
                    kv[4] = b.x; kv[5] = b.y; kv[6] = b.z; kv[7] = b.w;
                } else {
                    const uint4 u = *reinterpret_cast<const uint4*>(kr + d);
                    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        kv[2 * i] = __low2float(b2[i]);
                        kv[2 * i + 1] = __high2float(b2[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) dot = fmaf(qs[warp][d + i], kv[i], dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));      // at least one key of the chunk is valid
        const float alpha = expf(m - m_new);             // exp(-inf) = 0 on the first chunk
        const float pr = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int nk = min(32, p - c0 + 1);
        for (int j = 0; j < nk; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int kpj = c0 + j;
            if (kpj < first) continue;                     // uniform across the warp
            const int page = bt[kpj / page_size];
            const T* vr = v_pages + (((size_t)page * Hkv + hk) * page_size + kpj % page_size) * dh;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dh) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * dh;
    const float inv = 1.f / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dh) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

MLLM_EXPORT int mllm_attention_simt(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                    const int* block_table, int bt_stride, const int* token_seq,
                                    const int* positions, void* out, long long out_stride, int T, int H, int Hkv,
                                    int dh, int page_size, float scale, int window, int dtype,
                                    cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dh <= 0 || dh % 16 != 0 || dh > MAX_DH)
        return mllm_fail(1, "attention: head size %d is not a multiple of 16 in 16..%d", dh, MAX_DH);
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention: %d heads over %d key/value heads", H, Hkv);
    if (page_size <= 0) return mllm_fail(1, "attention: page size %d", page_size);
    const long long warps = (long long)T * H;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return mllm_fail(1, "attention: too many (token, head) pairs");
    if (dtype == MLLM_F32) {
        attention_simt_kernel<float><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table, bt_stride,
            token_seq, positions, (float*)out, out_stride, T, H, Hkv, dh, page_size, scale, window);
    } else if (dtype == MLLM_BF16) {
        using bf = __nv_bfloat16;
        attention_simt_kernel<bf><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
            (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride, token_seq,
            positions, (bf*)out, out_stride, T, H, Hkv, dh, page_size, scale, window);
    } else {
        return mllm_fail(1, "attention: unknown dtype code %d", dtype);
    }
    MLLM_CHECK_LAUNCH("attention_simt");
    return 0;
}
