// Copies the step's keys and values into their page slots.
// Source rows are column ranges of the fused QKV buffer (row stride given);
// destination layout per layer is [page][kv_head][offset][head_dim], so one
// (page, head) is one contiguous chunk.  slot = page * page_size + offset, the
// reference's token_to_block/token_to_offset pair merged
// (src/kernels/prefill/append_kv.cu:28-46; src/model/gpt2_model.cu:225-231).
#include "common.cuh"

template <typename T>
__global__ void kv_write_kernel(const T* k, const T* v, long long row_stride,
                                T* __restrict__ k_pages, T* __restrict__ v_pages,
                                const int* __restrict__ slots, int Hkv, int dh, int page_size) {
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch();
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot % page_size;
    const T* ks = k + (size_t)t * row_stride;
    const T* vs = v + (size_t)t * row_stride;
    const int n = Hkv * dh;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int h = i / dh, d = i % dh;
        const size_t dst = (((size_t)page * Hkv + h) * page_size + off) * dh + d;
        k_pages[dst] = ks[i];
        v_pages[dst] = vs[i];
    }
}

// The same copy in 16-byte pieces: a thread moves one piece of a key row and of a value row.
template <typename T>
__global__ void __launch_bounds__(256)
kv_write_vec_kernel(const T* k, const T* v, long long row_stride, T* __restrict__ k_pages,
                    T* __restrict__ v_pages, const int* __restrict__ slots, int T_tokens, int Hkv, int dh,
                    int page_size) {
    constexpr int VEC = 16 / sizeof(T);
    pdl_wait();
    pdl_launch();
    const int per = Hkv * dh / VEC;
    const long long total = (long long)T_tokens * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per), c = (int)(i % per);
        const int slot = slots[t];
        if (slot < 0) continue;
        const int e = c * VEC, h = e / dh, d = e % dh;
        const size_t dst = (((size_t)(slot / page_size) * Hkv + h) * page_size + slot % page_size) * dh + d;
        *reinterpret_cast<uint4*>(k_pages + dst) = *reinterpret_cast<const uint4*>(k + (size_t)t * row_stride + e);
        *reinterpret_cast<uint4*>(v_pages + dst) = *reinterpret_cast<const uint4*>(v + (size_t)t * row_stride + e);
    }
}

template <typename T>
static int kv_write_vec(const void* k, const void* v, long long row_stride, void* k_pages, void* v_pages,
                        const int* slots, int T_tokens, int Hkv, int dh, int page_size, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    const long long total = (long long)T_tokens * (Hkv * dh / VEC);
    const int grid = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    MLLM_CUDA(mllm_launch(kv_write_vec_kernel<T>, dim3(grid), dim3(256), 0, stream, true, (const T*)k, (const T*)v,
                          row_stride, (T*)k_pages, (T*)v_pages, slots, T_tokens, Hkv, dh, page_size));
    return 0;
}

MLLM_EXPORT int mllm_kv_write(const void* k, const void* v, long long row_stride, void* k_pages, void* v_pages,
                              const int* slots, int T, int Hkv, int dh, int page_size, int dtype,
                              cudaStream_t stream) {
    if (T <= 0) return 0;
    const int n = Hkv * dh;
    const int vec = dtype == MLLM_F32 ? 4 : 8;
    if ((dtype == MLLM_F32 || dtype == MLLM_BF16) && dh % vec == 0 && row_stride % vec == 0 && (uintptr_t)k % 16 == 0 &&
        (uintptr_t)v % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0) {
        if (dtype == MLLM_F32)
            return kv_write_vec<float>(k, v, row_stride, k_pages, v_pages, slots, T, Hkv, dh, page_size, stream);
        return kv_write_vec<__nv_bfloat16>(k, v, row_stride, k_pages, v_pages, slots, T, Hkv, dh, page_size, stream);
    }
    int threads = n >= 256 ? 256 : ((n + 31) / 32) * 32;
    if (dtype == MLLM_F32)
        kv_write_kernel<float><<<T, threads, 0, stream>>>((const float*)k, (const float*)v, row_stride,
                                                          (float*)k_pages, (float*)v_pages, slots, Hkv, dh, page_size);
    else if (dtype == MLLM_BF16)
        kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, row_stride, (__nv_bfloat16*)k_pages,
            (__nv_bfloat16*)v_pages, slots, Hkv, dh, page_size);
    else
        return mllm_fail(1, "kv_write: unknown dtype code %d", dtype);
    MLLM_CHECK_LAUNCH("kv_write");
    return 0;
}
