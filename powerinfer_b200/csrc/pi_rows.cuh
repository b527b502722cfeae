// Device helpers shared by the one-token sparse kernels: activity masks -> ranks of the active rows, the Q4_0 x Q8_0 block
// dot, packed FP32 FMAs.
#pragma once
#include "pi_common.cuh"

namespace pi {

static constexpr int QK = 32;
static constexpr int ROWS_THREADS = 512;
static constexpr int ROWS_WARPS = ROWS_THREADS / 32;
static constexpr int ROWS_MAX_CHUNKS = 4096;            // mask words one CTA scans (131072 neurons)
static constexpr int SLICE = 1024;                      // columns of an axpy slice: 32 sums per lane
static constexpr int AXPY_MAX_CTA_ROWS = 4096;          // rows one axpy CTA may own

// ---------------------------------------------------------------------------------------------- masks -> ranks
// s_mask[n_chunks], s_pref[n_chunks + 1] (exclusive prefix of popc), s_warp[ROWS_WARPS]: all in shared memory.
// Returns the number of active rows.  Ends with a block barrier.
static constexpr int SCAN_WORDS = ROWS_MAX_CHUNKS / ROWS_THREADS;   // mask words per thread

// first half: this thread's mask words into registers (an L2 round trip the caller can overlap with other loads)
__device__ __forceinline__ void scan_masks_load(const uint32_t * __restrict__ masks, int n_chunks, int nrows, uint32_t (&m)[SCAN_WORDS]) {
    const int per = (n_chunks + ROWS_THREADS - 1) / ROWS_THREADS;
    const int c0 = min((int)threadIdx.x * per, n_chunks), c1 = min(c0 + per, n_chunks);
#pragma unroll
    for (int k = 0; k < SCAN_WORDS; k++) {
        m[k] = 0u;
        if (c0 + k < c1) {
            m[k] = __ldcg(masks + c0 + k);
            const int left = nrows - (c0 + k) * 32;                 // bits beyond the last row never count
            if (left < 32) m[k] &= left <= 0 ? 0u : ((1u << left) - 1u);
        }
    }
}

// second half: block-wide exclusive scan of the popcounts
__device__ __forceinline__ int scan_masks_finish(const uint32_t (&m)[SCAN_WORDS], int n_chunks,
                                                 uint32_t * s_mask, int * s_pref, int * s_warp) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int per = (n_chunks + ROWS_THREADS - 1) / ROWS_THREADS;
    const int c0 = min(tid * per, n_chunks), c1 = min(c0 + per, n_chunks);
    int mine = 0;
#pragma unroll
    for (int k = 0; k < SCAN_WORDS; k++) mine += __popc(m[k]);
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[wid] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < wid; w++) base += s_warp[w];
    int off = base + incl - mine;
#pragma unroll
    for (int k = 0; k < SCAN_WORDS; k++) {
        if (c0 + k < c1) { s_mask[c0 + k] = m[k]; s_pref[c0 + k] = off; off += __popc(m[k]); }
    }
    if (tid == ROWS_THREADS - 1) s_pref[n_chunks] = base + incl;
    __syncthreads();
    return s_pref[n_chunks];
}

__device__ __forceinline__ int scan_masks(const uint32_t * __restrict__ masks, int n_chunks, int nrows,
                                          uint32_t * s_mask, int * s_pref, int * s_warp) {
    uint32_t m[SCAN_WORDS];
    scan_masks_load(masks, n_chunks, nrows, m);
    return scan_masks_finish(m, n_chunks, s_mask, s_pref, s_warp);
}

// local row number of the active row with rank `rank` (0 <= rank < total)
__device__ __forceinline__ int row_of_rank(int rank, int n_chunks, const uint32_t * s_mask, const int * s_pref) {
    int lo = 0, hi = n_chunks;                                      // largest c with s_pref[c] <= rank
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_pref[mid] <= rank) lo = mid; else hi = mid;
    }
    uint32_t m = s_mask[lo];
    for (int k = rank - s_pref[lo]; k > 0; k--) m &= m - 1;         // drop the k lowest set bits
    return lo * 32 + __ffs(m) - 1;
}

__device__ __forceinline__ int q4_block_dot(const uint4 q, const uint4 lo, const uint4 hi, int s8) {
    int sumi = 0;
    sumi = __dp4a((int)(q.x & 0x0F0F0F0Fu), (int)lo.x, sumi);
    sumi = __dp4a((int)((q.x >> 4) & 0x0F0F0F0Fu), (int)hi.x, sumi);
    sumi = __dp4a((int)(q.y & 0x0F0F0F0Fu), (int)lo.y, sumi);
    sumi = __dp4a((int)((q.y >> 4) & 0x0F0F0F0Fu), (int)hi.y, sumi);
    sumi = __dp4a((int)(q.z & 0x0F0F0F0Fu), (int)lo.z, sumi);
    sumi = __dp4a((int)((q.z >> 4) & 0x0F0F0F0Fu), (int)hi.z, sumi);
    sumi = __dp4a((int)(q.w & 0x0F0F0F0Fu), (int)lo.w, sumi);
    sumi = __dp4a((int)((q.w >> 4) & 0x0F0F0F0Fu), (int)hi.w, sumi);
    return sumi - 8 * s8;
}

__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    return (unsigned long long)__float_as_uint(a) | ((unsigned long long)__float_as_uint(b) << 32);
}
// two FP32 FMAs in one instruction (each lane rounds like fmaf)
__device__ __forceinline__ void ffma2(unsigned long long & acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
__device__ __forceinline__ float lo_f(unsigned long long v) { return __uint_as_float((unsigned)(v & 0xffffffffull)); }
__device__ __forceinline__ float hi_f(unsigned long long v) { return __uint_as_float((unsigned)(v >> 32)); }

}  // namespace pi
