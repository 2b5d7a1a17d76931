// Next-token choice on the device: argmax and temperature sampling over 32-bit logits.
//
// argmax: the lowest id among equal maxima, as the reference's argmax_rows_kernel
// (src/kernels/argmax.cu:12-20, 22-75).  Temperature: p = softmax(logits / T) in
// 32-bit and an inverse-CDF draw with a uniform number u in [0,1) that the host
// derives from (seed, request, index of the token), so a draw does not depend on
// what else is in the batch.  The cumulative sum runs in a fixed order: every thread
// owns one contiguous slice of the vocabulary, slices are summed left to right,
// then the slice sums are scanned in thread order.  Rows with T == 0 take the argmax.
#include "common.cuh"

namespace {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(256)
argmax_kernel(const float* logits, long long ld, int V, int* __restrict__ out) {
    __shared__ float bv[256];
    __shared__ int bi[256];
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = bv[threadIdx.x + s];
            const int oi = bi[threadIdx.x + s];
            if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) {
                bv[threadIdx.x] = ov;
                bi[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi[0] == 0x7fffffff ? 0 : bi[0];
}

// argmax of long rows with few rows in the batch: every row is cut into slices, one CTA
// each; the CTA that finishes a row last (a counter it resets) reduces the slices' results.
__global__ void __launch_bounds__(256)
argmax_sliced_kernel(const float* logits, long long ld, int V, int* __restrict__ out,
                     float* __restrict__ part_val, int* __restrict__ part_idx, unsigned int* __restrict__ counters) {
    __shared__ float bv[256];
    __shared__ int bi[256];
    __shared__ int s_last;
    pdl_wait();
    const int r = blockIdx.y, slices = gridDim.x, sl = blockIdx.x;
    const int per = (V + slices - 1) / slices;
    const int lo = min(V, sl * per), hi = min(V, lo + per);
    const float* row = logits + (size_t)r * ld;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float ov = bv[threadIdx.x + s];
            const int oi = bi[threadIdx.x + s];
            if (ov > bv[threadIdx.x] || (ov == bv[threadIdx.x] && oi < bi[threadIdx.x])) {
                bv[threadIdx.x] = ov;
                bi[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        part_val[(size_t)r * slices + sl] = bv[0];
        part_idx[(size_t)r * slices + sl] = bi[0];
        __threadfence();
        const unsigned int old = atomicAdd(&counters[r], 1u);
        s_last = old == (unsigned int)slices - 1;
        if (s_last) counters[r] = 0;
    }
    __syncthreads();
    if (!s_last || threadIdx.x != 0) return;
    __threadfence();
    float b = -INFINITY;
    int bidx = 0x7fffffff;
    for (int s = 0; s < slices; ++s) {
        const float v = __ldcg(&part_val[(size_t)r * slices + s]);
        const int i = __ldcg(&part_idx[(size_t)r * slices + s]);
        if (v > b || (v == b && i < bidx)) { b = v; bidx = i; }
    }
    out[r] = bidx == 0x7fffffff ? 0 : bidx;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* logits, long long ld, int V, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ float scratch[33];
    __shared__ float sums[SAMPLE_THREADS];
    __shared__ int s_idx;
    __shared__ int s_best;
    pdl_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temperature[r];
    const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);

    float best = -INFINITY;
    int bidx = 0x7fffffff;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v > best) { best = v; bidx = i; }          // ascending i: keeps the lowest id
    }
    const float mx = block_max(best, scratch);
    if (tid == 0) { s_idx = 0x7fffffff; s_best = 0x7fffffff; }
    __syncthreads();
    if (best == mx && bidx != 0x7fffffff) atomicMin(&s_best, bidx);
    __syncthreads();
    if (!(temp > 0.f)) {
        if (tid == 0) out[r] = s_best == 0x7fffffff ? 0 : s_best;
        return;
    }
    const float inv_t = 1.f / temp;
    float s = 0.f;
    for (int i = lo; i < hi; ++i) s += expf((row[i] - mx) * inv_t);
    sums[tid] = s;
    __syncthreads();
    // exclusive scan of the slice sums in thread order (Hillis-Steele on a copy is
    // order-dependent only through blockDim, which is fixed)
    float incl = s;
    for (int off = 1; off < SAMPLE_THREADS; off <<= 1) {
        const float add = tid >= off ? sums[tid - off] : 0.f;
        __syncthreads();
        incl += add;
        sums[tid] = incl;
        __syncthreads();
    }
    const float total = sums[SAMPLE_THREADS - 1];
    const float target = uniform[r] * total;
    const float excl = incl - s;
    if (hi > lo && incl > target && excl <= target) {
        float c = excl;
        int pick = hi - 1;
        for (int i = lo; i < hi; ++i) {
            c += expf((row[i] - mx) * inv_t);
            if (c > target) { pick = i; break; }
        }
        atomicMin(&s_idx, pick);
    }
    __syncthreads();
    if (tid == 0) out[r] = s_idx == 0x7fffffff ? (s_best == 0x7fffffff ? 0 : s_best) : s_idx;
}

}  // namespace

MLLM_EXPORT int mllm_argmax(const float* logits, long long ld, int R, int V, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return mllm_fail(1, "argmax: vocabulary %d", V);
    MLLM_CUDA(mllm_launch(argmax_kernel, dim3(R), dim3(256), 0, stream, true, logits, ld, V, out));
    return 0;
}

// Scratch: part_val/part_idx [R * slices], counters [R] zero before the first call (left zero).
MLLM_EXPORT int mllm_argmax_sliced(const float* logits, long long ld, int R, int V, int* out, float* part_val,
                                   int* part_idx, unsigned int* counters, int slices, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0 || slices <= 0 || R > 65535) return mllm_fail(1, "argmax: vocabulary %d, %d slices, %d rows", V, slices, R);
    MLLM_CUDA(mllm_launch(argmax_sliced_kernel, dim3(slices, R), dim3(256), 0, stream, true, logits, ld, V, out,
                          part_val, part_idx, counters));
    return 0;
}

MLLM_EXPORT int mllm_sample(const float* logits, long long ld, int R, int V, const float* temperature,
                            const float* uniform, int* out, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (V <= 0) return mllm_fail(1, "sample: vocabulary %d", V);
    MLLM_CUDA(mllm_launch(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, stream, true, logits, ld, V, temperature,
                          uniform, out));
    return 0;
}
