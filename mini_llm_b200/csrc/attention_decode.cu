// Attention of single tokens over the paged cache, split along the keys: the decode
// step's attention, where the time goes into reading keys and values once and, at small
// batches, into the latency of the chain position -> block table -> key/value rows.
//
// Grid (split, head, token).  A split is a fixed range of 128 key positions counted
// from position 0, so which keys are added together never depends on the batch.
// Inside a CTA (4 warps) a group of LPK lanes owns one key at a time: each lane takes
// 16 bytes of the key row and of the value row (the cache layout keeps one
// (page, head, slot) row contiguous).  With heads up to 64 a split's rows (or, with a
// 32-bit cache and a large grid, half a split's at a time) are first brought into shared
// memory by bulk copies, one per page (see Staged below); otherwise a group fetches the page ids of all its keys, then issues
// all its key and value loads at once (up to 8 keys in flight per group), and only
// then starts computing.  Either way it is three dependent memory round trips per CTA
// instead of two per key.  The group reduces each dot product with shuffles and keeps its
// own online-softmax state (m, l, o) in 32-bit (src/kernels/prefill/flashattention.cu:
// 129-168 gives the recurrence); groups are merged in group order through shared memory
// and the split's (m, l, o) goes to a scratch buffer.  The CTA that finishes last for a
// (token, head) - found with a counter that it resets - merges the splits in split order
// and divides by l, so one launch does it all.  The reference's decode kernel walks all
// keys with one thread per key and one thread per output element
// (src/kernels/decode/paged_attention.cu:60-120).
//
// When the CTAs of a (token, head) fit a thread-block cluster (up to 8) they are launched as
// one cluster and meet in distributed shared memory: every CTA leaves the (m, l, o) of its
// splits in its own shared memory, the CTA with the first split reads them over the
// SM-to-SM network in split order and writes the result; no scratch in global memory, no
// fence, no counter.  With few (token, head) pairs every split gets a CTA of its own; with
// many, a CTA walks up to 8 splits one after the other (the other resident CTAs hide its
// waits), down to one CTA per pair, which then needs no cluster at all.  The partial
// results and the order of their merge are the same in every arrangement, so a token's
// result does not depend on the size of the batch.  Longer contexts use the scratch path.
#include "common.cuh"
#include "tcgen05.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace {

constexpr int SPLIT = 128;
constexpr int MAX_CLUSTER = 8;
constexpr int THREADS = 128;

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[4]) {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y);
        v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[8]) {
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __low2float(b[i]);
            v[2 * i + 1] = __high2float(b[i]);
        }
    }
};

// acc + a.lo * b.lo + a.hi * b.hi for two packed pairs of bfloat16, each step one fused multiply-add whose
// product is exact and whose sum is rounded once to 32-bit.
__device__ __forceinline__ float dot2_bf16(uint32_t a, uint32_t b, float acc) {
    asm("{\n\t.reg .b16 a0, a1, b0, b1;\n\t"
        "mov.b32 {a0, a1}, %1;\n\t"
        "mov.b32 {b0, b1}, %2;\n\t"
        "fma.rn.f32.bf16 %0, a0, b0, %0;\n\t"
        "fma.rn.f32.bf16 %0, a1, b1, %0;\n\t}"
        : "+f"(acc) : "r"(a), "r"(b));
    return acc;
}

// How the splits of one (token, head) meet.
enum { MODE_SCRATCH = 0,     // partial results in global scratch; the CTA that arrives last merges them
       MODE_CLUSTER = 1,     // the CTAs of a (token, head) form a cluster and meet in distributed shared memory
       MODE_LOCAL = 2 };     // one CTA walks all the splits and merges them from its own shared memory

constexpr int MAX_SPC = 8;   // splits that one CTA may take, one after the other

// e^x for the softmax.  The 32-bit path keeps expf; with a bfloat16 cache the scores are kept in base 2
// (the query is scaled by log2 e as well) and one ex2.approx instruction, good to 2^-22, does it.
template <typename T> struct Exp;
template <> struct Exp<float> {
    static constexpr float QSCALE = 1.f;
    static __device__ __forceinline__ float of(float x) { return expf(x); }
};
template <> struct Exp<__nv_bfloat16> {
    static constexpr float QSCALE = 1.4426950408889634f;
    static __device__ __forceinline__ float of(float x) {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
};

// Keys and values of a split can be staged in shared memory when a split's rows fit there: heads up to 64
// (32 KB per CTA with a bfloat16 cache, 64 KB with a 32-bit one, or 32 KB there too with half a split staged at a time
// once the grid is large; dynamic shared memory).  The rows of one (page, head) are contiguous, so one thread brings each page's visible rows with one
// bulk copy (cp.async.bulk onto an mbarrier): no thread computes an address per key, no register is held while
// the rows fly, and six CTAs fit an SM instead of four.  That pays as soon as the grid is larger than about two
// CTAs per SM; smaller grids keep the rows in registers, one hop less on the way.  The arithmetic is the same
// either way.
__device__ int g_decode_error = 0;                   // 1: a staged split never arrived (bounded wait ran out)
template <typename T, int LPK> struct Staged {
    static constexpr bool value = LPK * Vec16<T>::N <= 64;                              // heads up to 64, either dtype
    static constexpr int BYTES = 2 * SPLIT * LPK * 16;                                  // a split's keys and values
    static constexpr int CTAS = BYTES <= 32 * 1024 ? 6 : 3;                             // resident CTAs per SM to aim for
};

// ONE: every CTA takes exactly one split.  STG: keys and values go through shared memory.  TWO: the staging area holds
// half a split (possible where the lane groups take a split's keys in two rounds of 64: 32-bit heads of 64): the
// halves are staged one after the other in the same 32 KB, so that six CTAs fit an SM instead of three.  Which keys
// meet in which order does not change.
template <typename T, int LPK, int MODE, bool ONE, bool STG, bool TWO = false>
__global__ void __launch_bounds__(THREADS, STG ? (TWO ? 6 : Staged<T, LPK>::CTAS) : 0)
attn_decode_kernel(const T* q, long long q_stride, const T* k_pages,      // written by kernels of this step: no __restrict__,
                   const T* v_pages,                                        // the compiler must not read them on the non-coherent path
                   const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ token_seq, const int* __restrict__ positions, T* __restrict__ out,
                   long long out_stride, float* __restrict__ part_o, float* __restrict__ part_ml,
                   unsigned int* __restrict__ counters, int H, int Hkv, int page_size, float scale, int window,
                   int max_splits, int spc_arg) {
    const int spc = ONE ? 1 : spc_arg;
    constexpr int VEC = Vec16<T>::N;
    constexpr int DH = LPK * VEC;
    constexpr int NG = THREADS / LPK;                 // key groups per CTA
    constexpr int KPG = SPLIT / NG;                   // keys per group in a split
    constexpr int UNR = KPG < 8 ? KPG : 8;            // keys in flight per group
    constexpr int RES = DH + 2;                       // a split's (o, m, l)
    // One split per CTA in a cluster: every CTA writes its (o, m, l) straight into the shared memory of the
    // CTA that merges, so the merge reads local memory only and the others may leave after one barrier.
    constexpr bool PUSH = MODE == MODE_CLUSTER && ONE;
    constexpr bool STAGE = STG;
    static_assert(!STG || Staged<T, LPK>::value, "a split's rows do not fit the staging area");
    static_assert(!TWO || (STG && NG * UNR * 2 == SPLIT), "two rounds of staging need groups that take a split in two rounds");
    constexpr int STAGE_KEYS = TWO ? SPLIT / 2 : SPLIT;       // keys that the staging area holds
    __shared__ float sm_m[NG], sm_l[NG], sm_w[NG];
    extern __shared__ __align__(16) uint4 s_stage[];          // STAGE: a split's keys, then its values: [key][16-byte piece]
    __shared__ float sm_o_own[STAGE ? 1 : NG * DH];
    float* sm_o = STAGE ? reinterpret_cast<float*>(s_stage) : sm_o_own;   // staged: the groups' outputs reuse the keys' space
    __shared__ float sm_res[(PUSH ? MAX_CLUSTER : MODE == MODE_SCRATCH || ONE ? 1 : MAX_SPC) * RES];
    __shared__ int s_last;
    __shared__ __align__(8) uint64_t s_bar;                   // STAGE: a split's bulk copies complete here
    const int cx = blockIdx.x, h = blockIdx.y, t = blockIdx.z;
    // Positions, the request index and the block table are written by the host before the step, and the rows of
    // all keys before the token's own position were written by earlier steps: all of that is read before the
    // wait on the previous kernel, which only brings the queries and the token's own key and value.
    // Everything read before the wait goes to L2 (ld.global.cg / cp.async.cg): a kernel that starts while its
    // predecessors still run finds whatever earlier kernels left in this SM's L1, and with rows shorter than a
    // cache line that can be a line fetched before a neighbouring row was written.
    pdl_launch();
    const int p = __ldcg(positions + t);
    const int seq = __ldcg(token_seq + t);
    int first = 0;
    if (window > 0 && p - window + 1 > 0) first = p - window + 1;
    const int s_lo = first / SPLIT, s_hi = p / SPLIT;         // splits that have work, inclusive
    // this CTA takes the splits cx*spc .. cx*spc+spc-1, one after the other
    const int my_lo = max(cx * spc, s_lo), my_hi = min(cx * spc + spc - 1, s_hi);
    const bool single = s_lo == s_hi;                         // the only split: its result is the output
    const int c_lo = spc == 1 ? s_lo : s_lo / spc, c_hi = spc == 1 ? s_hi : s_hi / spc;   // CTAs with work
    const bool several = c_lo != c_hi;                        // more than one (the same answer in all of them)
    if (my_lo > my_hi) {                                      // nothing visible for this CTA
        if constexpr (MODE == MODE_CLUSTER) {
            if (several) {                                    // the others still meet at the cluster's barriers
                cg::cluster_group cluster = cg::this_cluster();
                cluster.sync();
                cluster.sync();
            }
        }
        return;
    }
    if constexpr (PUSH) {
        // first barrier, arrival only: once it completes every CTA of the cluster runs and its shared memory
        // may be written; it is waited for just before the results go out, long after it has completed
        if (several) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    }
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int gi = threadIdx.x / LPK, li = threadIdx.x % LPK;
    // page sizes are powers of two in practice: a shift and a mask instead of two divisions per key
    const bool pow2 = (page_size & (page_size - 1)) == 0;
    const int pshift = __ffs(page_size) - 1, pmask = page_size - 1;
    auto page_index = [&](int kp) { return pow2 ? kp >> pshift : kp / page_size; };
    auto page_offset = [&](int kp) { return pow2 ? kp & pmask : kp % page_size; };

    constexpr bool MIXED = STAGE && sizeof(T) == 2;           // scores from the packed query and keys, scaled afterwards
    uint4 qw = make_uint4(0, 0, 0, 0);
    float qv[VEC];                                            // loaded after the wait, in the first split's turn
    bool waited = false;
    const size_t pair = (size_t)t * H + h;
    uint32_t phase = 0;
    if constexpr (STAGE) {
        if (threadIdx.x == 0) {
            tc::mbar_init(&s_bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }
    // the wait on the previous kernel, then this thread's part of the query
    auto wait_and_load_q = [&]() {
        pdl_wait();
        waited = true;
        // (what the previous kernel wrote is read past L1)
        const uint4 qraw = __ldcg(reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)h * DH + li * VEC));
        qw = qraw;
        Vec16<T>::unpack(qraw, qv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) qv[i] *= scale * Exp<T>::QSCALE;
    };

    // Asks for the rows of the keys [lo, hi) that this CTA will come to (visible ones only) to be brought into L2, one
    // key per thread.
    auto ask_for = [&](int lo, int hi) {
        constexpr int ROW_BYTES = DH * (int)sizeof(T);
        hi = min(hi, min((my_hi + 1) * SPLIT, p + 1));
        for (int kp = max(lo, first) + (int)threadIdx.x; kp < hi; kp += THREADS) {
            const size_t off = (((size_t)__ldcg(bt + page_index(kp)) * Hkv + hk) * page_size + page_offset(kp)) * DH;
#pragma unroll
            for (int b = 0; b < ROW_BYTES; b += 128) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(k_pages + off) + b));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(v_pages + off) + b));
            }
        }
    };
    // Only CTAs that load rows straight into registers ask for later splits ahead of time (the next one now, each later
    // one two splits before its turn).  With staging through shared memory the bulk copies of the resident CTAs keep
    // HBM busy by themselves, and asking ahead made every large grid slower: all later splits at once evicted each
    // other from L2 (274 MB read for 201 MB of cache at batch 64), two rounds ahead still cost 7-8 % against none
    // (39.5 against 36.5 us in float32, 22.7 against 22.0 us in bfloat16 at batch 64).
    if constexpr (!ONE && !STAGE) ask_for((my_lo + 1) * SPLIT, (my_lo + 2) * SPLIT);

#pragma unroll 1
    for (int split = my_lo; split <= my_hi; ++split) {
        const int k_lo = split * SPLIT, k_hi = min(k_lo + SPLIT, p + 1);
        float m = -INFINITY, l = 0.f, o[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = 0.f;
        uint4* sk = s_stage;
        uint4* sv = s_stage + STAGE_KEYS * LPK;
        // Brings the visible rows of [lo, hi) into the staging area (row r to place r - lo), page by page: thread c
        // brings the rows of the c-th page that the range touches.  Rows of earlier steps go out before the wait on
        // the previous kernel, the token's own row (position p) after it.  Rows that are not visible are not
        // copied: their places hold whatever was there, and the arithmetic below skips them.
        auto stage = [&](int lo, int hi) {
            constexpr uint32_t ROW = DH * (uint32_t)sizeof(T);
            const int v_lo = max(lo, first);
            const int pre_hi = min(hi, p);
            if (threadIdx.x == 0) tc::mbar_expect_tx(&s_bar, (uint32_t)max(0, hi - v_lo) * ROW * 2);
            if (pre_hi > v_lo) {
                const int pg0 = page_index(v_lo), pg1 = page_index(pre_hi - 1);
                for (int pg = pg0 + (int)threadIdx.x; pg <= pg1; pg += THREADS) {
                    const int r0 = max(v_lo, pg * page_size), r1 = min(pre_hi, (pg + 1) * page_size);
                    const size_t off = (((size_t)__ldcg(bt + pg) * Hkv + hk) * page_size + (r0 - pg * page_size)) * DH;
                    const uint32_t bytes = (uint32_t)(r1 - r0) * ROW;
                    tc::bulk_load(sk + (r0 - lo) * LPK, k_pages + off, bytes, &s_bar);
                    tc::bulk_load(sv + (r0 - lo) * LPK, v_pages + off, bytes, &s_bar);
                }
            }
            if (!waited) wait_and_load_q();
            if (threadIdx.x == 0 && p >= v_lo && p < hi) {
                const size_t off = (((size_t)__ldcg(bt + page_index(p)) * Hkv + hk) * page_size + page_offset(p)) * DH;
                tc::bulk_load(sk + (p - lo) * LPK, k_pages + off, ROW, &s_bar);
                tc::bulk_load(sv + (p - lo) * LPK, v_pages + off, ROW, &s_bar);
            }
            if (!tc::mbar_wait(&s_bar, phase)) {              // gave up: tell the host, let copies in flight land, go on
                if (threadIdx.x == 0) { atomicCAS(&g_decode_error, 0, 1); tc::report_to_host(301); }
                for (int i = 0; i < 2000; ++i) __nanosleep(100);
            }
            phase ^= 1;
        };
        if constexpr (STAGE && !TWO) stage(k_lo, k_hi);
        if constexpr (!ONE && !STAGE) ask_for((split + 2) * SPLIT, (split + 3) * SPLIT);
#pragma unroll 1
        for (int kb = k_lo + gi; kb < k_lo + SPLIT; kb += NG * UNR) {   // same trip count for every lane
            const int s_base = TWO ? kb - gi : k_lo;          // the key whose row lies first in the staging area
            if constexpr (TWO) {
                if (s_base > k_lo) {                          // second round: every group has left the first half
                    tc::fence_async_smem();
                    __syncthreads();
                }
                stage(s_base, min(s_base + STAGE_KEYS, k_hi));
            }
            bool ok[UNR];
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int kp = kb + u * NG;
                ok[u] = kp < k_hi && kp >= first;
            }
            uint4 kr[STAGE ? 1 : UNR], vr[STAGE ? 1 : UNR];
            if constexpr (!STAGE) {
                int page[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) page[u] = ok[u] ? __ldcg(bt + page_index(kb + u * NG)) : 0;
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {        // pass 0: the keys of earlier steps; pass 1, after the wait: the token's own
                    if (pass == 1 && !waited) wait_and_load_q();
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
                        const int kp = kb + u * NG;
                        if ((kp == p) != (pass == 1)) continue;
                        kr[u] = make_uint4(0, 0, 0, 0);
                        vr[u] = make_uint4(0, 0, 0, 0);
                        if (ok[u]) {
                            const size_t off = (((size_t)page[u] * Hkv + hk) * page_size + page_offset(kp)) * DH + li * VEC;
                            kr[u] = __ldcg(reinterpret_cast<const uint4*>(k_pages + off));
                            vr[u] = __ldcg(reinterpret_cast<const uint4*>(v_pages + off));
                        }
                    }
                }
            }
            float s[UNR];
            float mx = m;
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                float d = 0.f;
                if constexpr (MIXED) {
                    // bfloat16 x bfloat16 + 32-bit in one instruction: the products are exact, nothing is unpacked
                    const uint4 kw = sk[(kb + u * NG - s_base) * LPK + li];
                    d = dot2_bf16(qw.x, kw.x, d);
                    d = dot2_bf16(qw.y, kw.y, d);
                    d = dot2_bf16(qw.z, kw.z, d);
                    d = dot2_bf16(qw.w, kw.w, d);
                } else {
                    float kv[VEC];
                    if constexpr (STAGE) Vec16<T>::unpack(sk[(kb + u * NG - s_base) * LPK + li], kv);
                    else Vec16<T>::unpack(kr[u], kv);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) d = fmaf(qv[i], kv[i], d);
                }
#pragma unroll
                for (int off = LPK / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
                if constexpr (MIXED) d *= scale * Exp<T>::QSCALE;
                s[u] = ok[u] ? d : -INFINITY;
                mx = fmaxf(mx, s[u]);
            }
            if (mx != -INFINITY) {                               // uniform within the group; no shuffles inside
                const float alpha = Exp<T>::of(m - mx);
                l *= alpha;
#pragma unroll
                for (int i = 0; i < VEC; ++i) o[i] *= alpha;
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    if (STAGE && !ok[u]) continue;            // nothing was copied to this key's place
                    const float pr = ok[u] ? Exp<T>::of(s[u] - mx) : 0.f;
                    float vv[VEC];
                    if constexpr (STAGE) Vec16<T>::unpack(sv[(kb + u * NG - s_base) * LPK + li], vv);
                    else Vec16<T>::unpack(vr[u], vv);
                    l += pr;
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] = fmaf(pr, vv[i], o[i]);
                }
                m = mx;
            }
        }
        // the groups of the CTA are merged in group order
        if constexpr (STAGE) __syncthreads();                 // every group has read its keys: their space takes the outputs
        if (li == 0) { sm_m[gi] = m; sm_l[gi] = l; }
#pragma unroll
        for (int i = 0; i < VEC; ++i) sm_o[gi * DH + li * VEC + i] = o[i];
        __syncthreads();
        float M = -INFINITY;
        for (int g = 0; g < NG; ++g) M = fmaxf(M, sm_m[g]);
        if (threadIdx.x < NG)                                 // every group's weight in the merge, computed once
            sm_w[threadIdx.x] = sm_m[threadIdx.x] == -INFINITY ? 0.f : Exp<T>::of(sm_m[threadIdx.x] - M);
        __syncthreads();
        float L = 0.f;
        for (int g = 0; g < NG; ++g) L = fmaf(sm_w[g], sm_l[g], L);
        const size_t slot = pair * max_splits + split;
        float* res = sm_res + (MODE == MODE_SCRATCH ? 0 : (split - cx * spc) * RES);
        if constexpr (PUSH) {
            if (several) {
                asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                res = cg::this_cluster().map_shared_rank(sm_res, c_lo) + cx * RES;      // slot `split` of the merging CTA
            }
        }
        for (int d = threadIdx.x; d < DH; d += THREADS) {
            float acc = 0.f;
            for (int g = 0; g < NG; ++g) acc = fmaf(sm_w[g], sm_o[g * DH + d], acc);
            if (single) out[(size_t)t * out_stride + (size_t)h * DH + d] = from_f32<T>(acc / L);
            else if (MODE == MODE_SCRATCH) part_o[slot * DH + d] = acc;
            else res[d] = acc;
        }
        if (!single && threadIdx.x == 0) {
            if (MODE == MODE_SCRATCH) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
            else { res[DH] = M; res[DH + 1] = L; }
        }
        if (split < my_hi) {
            if constexpr (STAGE) tc::fence_async_smem();      // the next split's copies overwrite what was written here
            __syncthreads();                                  // the group buffers are free for the next split
        }
    }
    if (single) return;

    if constexpr (MODE != MODE_SCRATCH) {
        // every split's (o, m, l) stays in the shared memory of the CTA that computed it; the CTA with the
        // first split collects them in split order - over the SM-to-SM network where another CTA holds them
        cg::cluster_group cluster = cg::this_cluster();
        const bool remote = MODE == MODE_CLUSTER && several && !PUSH;
        if (PUSH) {
            cluster.sync();                                   // second barrier: every split's result has arrived
            if (cx != c_lo) return;
        } else if (remote) {
            cluster.sync();                                   // every split's result is in place
        } else {
            __syncthreads();
        }
        if (cx == c_lo) {
            // walks the splits s_lo..s_hi: CTA c holds the splits c*spc .. c*spc+spc-1 in that order
            auto held_by = [&](int c) -> const float* {
                if (PUSH) return sm_res + c * RES;            // pushed here, one slot per CTA
                return (remote && c <= c_hi) ? cluster.map_shared_rank(sm_res, c) : sm_res;
            };
            const int i_lo = s_lo - c_lo * spc;               // index of the first split inside its CTA
#define MLLM_NEXT_SPLIT(r, c, i)                                  \
    do {                                                          \
        if (++i == spc) { i = 0; ++c; r = held_by(c); }           \
        else r += RES;                                            \
    } while (0)
            float MM = -INFINITY;
            {
                int c = c_lo, i = i_lo;
                const float* r = held_by(c) + i * RES;
                for (int s = s_lo; s <= s_hi; ++s) {
                    MM = fmaxf(MM, r[DH]);
                    MLLM_NEXT_SPLIT(r, c, i);
                }
            }
            float LL = 0.f;
            {
                int c = c_lo, i = i_lo;
                const float* r = held_by(c) + i * RES;
                for (int s = s_lo; s <= s_hi; ++s) {
                    LL = fmaf(Exp<T>::of(r[DH] - MM), r[DH + 1], LL);
                    MLLM_NEXT_SPLIT(r, c, i);
                }
            }
            const float inv = 1.f / LL;
            for (int d = threadIdx.x; d < DH; d += THREADS) {
                float acc = 0.f;
                int c = c_lo, i = i_lo;
                const float* r = held_by(c) + i * RES;
                for (int s = s_lo; s <= s_hi; ++s) {
                    acc = fmaf(Exp<T>::of(r[DH] - MM), r[d], acc);
                    MLLM_NEXT_SPLIT(r, c, i);
                }
                out[(size_t)t * out_stride + (size_t)h * DH + d] = from_f32<T>(acc * inv);
            }
#undef MLLM_NEXT_SPLIT
        }
        if (remote) cluster.sync();                           // nobody leaves while its memory may be read
        return;
    }
    // the CTA that arrives last merges the splits of this (token, head)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int n = (unsigned int)(c_hi - c_lo + 1);
        const unsigned int old = atomicAdd(&counters[pair], 1u);
        s_last = (old == n - 1);
        if (s_last) counters[pair] = 0;                      // ready for the next launch
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t base = pair * max_splits;
    float MM = -INFINITY;
    for (int s = s_lo; s <= s_hi; ++s) MM = fmaxf(MM, __ldcg(&part_ml[(base + s) * 2]));
    float LL = 0.f;
    for (int s = s_lo; s <= s_hi; ++s)
        LL = fmaf(Exp<T>::of(__ldcg(&part_ml[(base + s) * 2]) - MM), __ldcg(&part_ml[(base + s) * 2 + 1]), LL);
    const float inv = 1.f / LL;
    for (int d = threadIdx.x; d < DH; d += THREADS) {
        float acc = 0.f;
        for (int s = s_lo; s <= s_hi; ++s)
            acc = fmaf(Exp<T>::of(__ldcg(&part_ml[(base + s) * 2]) - MM), __ldcg(&part_o[(base + s) * DH + d]), acc);
        out[(size_t)t * out_stride + (size_t)h * DH + d] = from_f32<T>(acc * inv);
    }
}

int g_last_staging = 0;   // how the most recent launch staged keys and values: 0 not, 1 a split at a time, 2 half a split

int decode_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <typename T, int LPK>
int launch(const void* q, long long q_stride, const void* k_pages, const void* v_pages, const int* block_table,
           int bt_stride, const int* token_seq, const int* positions, void* out, long long out_stride,
           float* part_o, float* part_ml, unsigned int* counters, int T_tokens, int H, int Hkv, int page_size,
           float scale, int window, int max_splits, bool scratch_path, cudaStream_t stream) {
    // CTAs per (token, head): few requests get one CTA per split, so that the chain position -> block table ->
    // rows is as short as it can be; many requests let a CTA walk several splits, which keeps the number of
    // CTAs near four per SM-slot instead of growing with the batch.  Which keys are added together, and in
    // which order, is the same either way.
    const long long pairs = (long long)T_tokens * H;
    long long want = (4LL * decode_sm_count() + pairs - 1) / pairs;
    int ctas = (int)(want < 1 ? 1 : (want > max_splits ? max_splits : want));
    // measured: one split per CTA stays ahead until the grid reaches about 24 CTAs per SM
    if (max_splits <= MAX_CLUSTER && pairs * max_splits <= 24LL * decode_sm_count()) ctas = max_splits;
    int spc = (max_splits + ctas - 1) / ctas;
    if (spc > MAX_SPC) spc = MAX_SPC;
    ctas = (max_splits + spc - 1) / spc;
    dim3 grid(ctas, H, T_tokens);
#define ARGS (const T*)q, q_stride, (const T*)k_pages, (const T*)v_pages, block_table, bt_stride, token_seq, positions, \
             (T*)out, out_stride, part_o, part_ml, counters, H, Hkv, page_size, scale, window, max_splits, spc
    using K = void (*)(const T*, long long, const T*, const T*, const int*, int, const int*, const int*, T*, long long,
                       float*, float*, unsigned int*, int, int, int, float, int, int, int);
    constexpr bool CAN_STAGE = Staged<T, LPK>::value;
    // staged whenever the rows fit (measured: never slower, from two requests on faster); bulk copies want
    // 16-byte aligned pools
    const bool stg = CAN_STAGE && ((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0;
    const int mode = scratch_path ? MODE_SCRATCH : ctas == 1 ? MODE_LOCAL : ctas <= MAX_CLUSTER ? MODE_CLUSTER : MODE_SCRATCH;
    const bool one = spc == 1 && mode != MODE_LOCAL;
    K kern;
    // Half a split staged at a time (32-bit heads of 64) lets six CTAs share an SM instead of three, at the price of a
    // second round of copies per split.  Measured at contexts of 520 and 1,000: it loses while the whole-split CTAs
    // still fit the SMs at once (5.3 against 6.4 us at 240 CTAs, 6.0 against 7.4 us at 300, 6.6 against 7.9 us at 360)
    // and wins beyond (8.7 against 8.2 us at 384 CTAs in clusters of 8, 10.3 against 8.5 us at 480, where 96 clusters
    // of 5 with 64 KB each need a second wave; 54 against 36 us with one CTA for each of 768 pairs): from two and a
    // half CTAs per SM on.  The bits are the same either way.
    constexpr bool CAN_TWO = CAN_STAGE && Staged<T, LPK>::BYTES > 32 * 1024 && LPK == 16 && sizeof(T) == 4;
    const bool two = CAN_TWO && stg && 2 * pairs * ctas > 5LL * decode_sm_count();
    g_last_staging = two ? 2 : stg ? 1 : 0;
#define PICK(M, O)                                                                     \
    kern = two ? (K)attn_decode_kernel<T, LPK, M, O, CAN_TWO, CAN_TWO>                 \
         : stg ? (K)attn_decode_kernel<T, LPK, M, O, CAN_STAGE> : (K)attn_decode_kernel<T, LPK, M, O, false>
    if (mode == MODE_LOCAL) PICK(MODE_LOCAL, false);
    else if (mode == MODE_CLUSTER && one) PICK(MODE_CLUSTER, true);
    else if (mode == MODE_CLUSTER) PICK(MODE_CLUSTER, false);
    else if (one) PICK(MODE_SCRATCH, true);
    else PICK(MODE_SCRATCH, false);
#undef PICK
    const size_t smem = stg ? (size_t)Staged<T, LPK>::BYTES / (two ? 2 : 1) : 0;
    if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (mode == MODE_CLUSTER) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = ctas;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_mllm_pdl ? 2 : 1;
        MLLM_CUDA(cudaLaunchKernelEx(&cfg, kern, ARGS));
        return 0;
    }
    MLLM_CUDA(mllm_launch(kern, grid, dim3(THREADS), smem, stream, true, ARGS));
#undef ARGS
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_attention_decode_split_len() { return SPLIT; }

// How the most recent launch of this file's kernel staged keys and values in shared memory: 0 not at all, 1 a split at a
// time, 2 half a split at a time (for tests of the arrangements).
MLLM_EXPORT int mllm_attention_decode_last_staging() { return g_last_staging; }

// The pinned host word that this file's kernels write when they give up on a wait.
MLLM_EXPORT int mllm_attention_decode_bind_error(int* word) { return tc::bind_host_error(word); }

// The first error recorded by the kernel since the last call (0 = none); resets it.
MLLM_EXPORT int mllm_attention_decode_error(int* code) {
    int zero = 0;
    MLLM_CUDA(cudaMemcpyFromSymbol(code, g_decode_error, sizeof(int)));
    if (*code) MLLM_CUDA(cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(int)));
    return 0;
}

// Everything a raw C caller can get wrong is refused here, on the host, before any launch and before any
// CUDA call: a bad size would index outside the pools on the device, a misaligned pool would fault in the
// 16-byte loads.  Returns 0 when the arguments can be launched.
static int attention_decode_check(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                  const int* block_table, int bt_stride, const int* token_seq, const int* positions,
                                  const void* out, int T, int H, int Hkv, int dh, int page_size, int window,
                                  int max_splits, int dtype) {
    if (T <= 0) return 0;
    if (!q || !k_pages || !v_pages || !block_table || !token_seq || !positions || !out)
        return mllm_fail(1, "attention_decode: null pointer among the inputs or the output");
    if (H <= 0 || Hkv <= 0 || H % Hkv != 0)
        return mllm_fail(1, "attention_decode: %d heads over %d key/value heads", H, Hkv);
    if (page_size <= 0) return mllm_fail(1, "attention_decode: page size %d", page_size);
    if (window < 0) return mllm_fail(1, "attention_decode: window %d (0 means all keys)", window);
    if (bt_stride <= 0) return mllm_fail(1, "attention_decode: block table row stride %d", bt_stride);
    if (max_splits <= 0 || T > 65535 || H > 65535) return mllm_fail(1, "attention_decode: grid out of range");
    if (dtype != MLLM_BF16 && dtype != MLLM_F32) return mllm_fail(1, "attention_decode: unknown dtype code %d", dtype);
    if (dh < 16 || dh > (dtype == MLLM_BF16 ? 256 : 128) || (dh & (dh - 1)))
        return mllm_fail(1, "attention_decode: head size %d is not one of this kernel's", dh);
    if (((uintptr_t)k_pages | (uintptr_t)v_pages) % 16)
        return mllm_fail(1, "attention_decode: the key and value pools must be 16-byte aligned");
    if (q_stride % (dtype == MLLM_BF16 ? 8 : 4) || (uintptr_t)q % 16)
        return mllm_fail(1, "attention_decode: queries must be 16-byte aligned");
    return 0;
}

static int attention_decode_impl(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                 const int* block_table, int bt_stride, const int* token_seq, const int* positions,
                                 void* out, long long out_stride, float* part_o, float* part_ml,
                                 unsigned int* counters, int T, int H, int Hkv, int dh, int page_size, float scale,
                                 int window, int max_splits, int dtype, bool scratch_path, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (int rc = attention_decode_check(q, q_stride, k_pages, v_pages, block_table, bt_stride, token_seq, positions, out,
                                        T, H, Hkv, dh, page_size, window, max_splits, dtype))
        return rc;
    if ((scratch_path || max_splits > 8) && (!part_o || !part_ml || !counters))
        return mllm_fail(1, "attention_decode: %d splits need the scratch buffers", max_splits);
#define GO(TT, LPK)                                                                                            \
    return launch<TT, LPK>(q, q_stride, k_pages, v_pages, block_table, bt_stride, token_seq, positions, out,    \
                           out_stride, part_o, part_ml, counters, T, H, Hkv, page_size, scale, window,          \
                           max_splits, scratch_path, stream)
    if (dtype == MLLM_BF16) {
        using bf = __nv_bfloat16;
        if (q_stride % 8 || (uintptr_t)q % 16) return mllm_fail(1, "attention_decode: queries must be 16-byte aligned");
        switch (dh) {
            case 16: GO(bf, 2);
            case 32: GO(bf, 4);
            case 64: GO(bf, 8);
            case 128: GO(bf, 16);
            case 256: GO(bf, 32);
        }
    } else if (dtype == MLLM_F32) {
        if (q_stride % 4 || (uintptr_t)q % 16) return mllm_fail(1, "attention_decode: queries must be 16-byte aligned");
        switch (dh) {
            case 16: GO(float, 4);
            case 32: GO(float, 8);
            case 64: GO(float, 16);
            case 128: GO(float, 32);
        }
    } else {
        return mllm_fail(1, "attention_decode: unknown dtype code %d", dtype);
    }
#undef GO
    return mllm_fail(1, "attention_decode: head size %d is not one of this kernel's", dh);
}

// Scratch (used when max_splits > 8 or scratch_only != 0): part_o [T*H*max_splits*dh] and
// part_ml [T*H*max_splits*2] floats and counters [T*H] 32-bit words that must be zero before
// the first call (the kernel leaves them zero).  The caller guarantees max_splits >=
// ceil((largest position + 1) / 128): a token whose keys need more splits than that gets no
// output written (positions live on the device, so the host cannot check this).  Sizes, null
// pointers and alignments are checked on the host and refused with code 1 before any launch.  With up to 8 splits the splits meet in a thread-block cluster instead and the
// scratch is not touched.  Fails for head sizes this kernel does not take (the caller then
// uses the general kernel).
MLLM_EXPORT int mllm_attention_decode(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                      const int* block_table, int bt_stride, const int* token_seq,
                                      const int* positions, void* out, long long out_stride, float* part_o,
                                      float* part_ml, unsigned int* counters, int T, int H, int Hkv, int dh,
                                      int page_size, float scale, int window, int max_splits, int dtype,
                                      int scratch_only, cudaStream_t stream) {
    return attention_decode_impl(q, q_stride, k_pages, v_pages, block_table, bt_stride, token_seq, positions, out,
                                 out_stride, part_o, part_ml, counters, T, H, Hkv, dh, page_size, scale, window,
                                 max_splits, dtype, scratch_only != 0, stream);
}

// ---------------------------------------------------------------------------------------
// The same attention for callers that cannot allocate device memory (declared in
// attention_decode_noalloc.h, which says who they are).  Its scratch - the per-split partial
// results and the per-(token, head) arrival counters - lives in this file-scope device array
// instead of in buffers that the caller provides.  Every GPU that loads the library carries
// the array until the process exits.
#include "attention_decode_noalloc.h"

namespace {

constexpr size_t NA_PART_O = (size_t)MLLM_NOALLOC_MAX_SLOTS * MLLM_NOALLOC_MAX_HEAD_DIM * sizeof(float);
constexpr size_t NA_PART_ML = (size_t)MLLM_NOALLOC_MAX_SLOTS * 2 * sizeof(float);
constexpr size_t NA_COUNTERS = (size_t)MLLM_NOALLOC_MAX_SLOTS * sizeof(unsigned int);
constexpr size_t NA_TOTAL = NA_PART_O + NA_PART_ML + NA_COUNTERS;

static __device__ __align__(256) unsigned char g_noalloc_scratch[NA_TOTAL];

constexpr int NA_MAX_DEVICES = 64;
unsigned char* g_noalloc_ptr[NA_MAX_DEVICES] = {};       // device address of the array, per device

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel could use: the device address has to be asked for, once per device, with that
// device current.
int noalloc_scratch(unsigned char** out) {
    int dev = -1;
    MLLM_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NA_MAX_DEVICES) return mllm_fail(1, "attention_decode_noalloc: device index %d", dev);
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return mllm_fail(3, "attention_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_attention_decode_noalloc(const void* q, long long q_stride, const void* k_pages,
                                              const void* v_pages, const int* block_table, int bt_stride,
                                              const int* token_seq, const int* positions, void* out,
                                              long long out_stride, int T, int H, int Hkv, int dh, int page_size,
                                              float scale, int window, int max_splits, int dtype,
                                              cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || max_splits <= 0) return mllm_fail(1, "attention_decode_noalloc: %d heads, %d splits", H, max_splits);
    const long long slots = (long long)T * H * max_splits;
    if (slots > MLLM_NOALLOC_MAX_SLOTS)
        return mllm_fail(1, "attention_decode_noalloc: tokens x heads x splits = %d x %d x %d = %lld exceeds the "
                            "built-in scratch of %d; use mllm_attention_decode with your own buffers",
                         T, H, max_splits, slots, MLLM_NOALLOC_MAX_SLOTS);
    if (dh > MLLM_NOALLOC_MAX_HEAD_DIM)
        return mllm_fail(1, "attention_decode_noalloc: head size %d exceeds %d", dh, MLLM_NOALLOC_MAX_HEAD_DIM);
    if (int rc = attention_decode_check(q, q_stride, k_pages, v_pages, block_table, bt_stride, token_seq, positions, out,
                                        T, H, Hkv, dh, page_size, window, max_splits, dtype))
        return rc;
    unsigned char* base = nullptr;
    const int rc = noalloc_scratch(&base);
    if (rc) return rc;
    float* part_o = reinterpret_cast<float*>(base);
    float* part_ml = reinterpret_cast<float*>(base + NA_PART_O);
    unsigned int* counters = reinterpret_cast<unsigned int*>(base + NA_PART_O + NA_PART_ML);
    // The array keeps what the last call left.  The partial results are fully rewritten before
    // they are read; the counters must start at zero, so they are cleared on this stream.
    MLLM_CUDA(cudaMemsetAsync(counters, 0, (size_t)T * H * sizeof(unsigned int), stream));
    return attention_decode_impl(q, q_stride, k_pages, v_pages, block_table, bt_stride, token_seq, positions, out,
                                 out_stride, part_o, part_ml, counters, T, H, Hkv, dh, page_size, scale, window,
                                 max_splits, dtype, /*scratch_path=*/true, stream);
}
