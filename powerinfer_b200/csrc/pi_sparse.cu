// The neuron-sparse half of the FFN: predictor mask -> compacted active list (warp ballot / popc), and the
// scatter-accumulate behind ggml_axpy over the rows of ffn_down_t named by that list.
#include "pi_common.cuh"

namespace pi {

static constexpr int QK = 32;

// ------------------------------------------------------------------------------------------------
// Compaction.  Phase A (all CTAs): one warp per 32 consecutive local rows; a lane tests its row for every token,
// __ballot_sync gives the 32-bit activity mask of the chunk.  Phase B (the CTA that finishes last, found with a
// ticket counter): exclusive scan of popc(mask) over the chunks and expansion into a SORTED list of local rows.
// No CTA ever waits for another one.  The ticket counter is left at zero for the next launch.
static constexpr int COMPACT_THREADS = 256;

struct CompactP {
    const float * idx; int64_t idx_stride; int T; float threshold;
    int n_local; const int32_t * bucket;
    int32_t * list; int32_t * count;
    uint32_t * masks; unsigned int * ticket;
    float * zero_dst; int64_t zero_stride;
    const float * fill_bias; int fill_relu;
    unsigned long long * total;
};

__global__ void __launch_bounds__(COMPACT_THREADS) k_compact(const CompactP p) {
    __shared__ int s_last;
    __shared__ int s_warp_sums[COMPACT_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31;
    const int n_chunks = (p.n_local + 31) / 32;
    const int warps_total = gridDim.x * (COMPACT_THREADS / 32);
    pdl_launch();
    pdl_wait();
    int n_act = 0;
    for (int c = blockIdx.x * (COMPACT_THREADS / 32) + (tid >> 5); c < n_chunks; c += warps_total) {
        const int r = c * 32 + lane;
        bool any = false;
        if (r < p.n_local) {
            const int64_t g = p.bucket ? p.bucket[r] : r;
            float fill = 0.f;
            if (p.zero_dst && p.fill_bias) { fill = p.fill_bias[g]; if (p.fill_relu) fill = fmaxf(fill, 0.f); }
            for (int t = 0; t < p.T; t++) {
                const bool a = !(p.idx[(size_t)t * p.idx_stride + g] < p.threshold);   // the reference skips on `<`: a NaN logit counts as active
                any |= a;
                if (p.zero_dst && !a) p.zero_dst[(size_t)t * p.zero_stride + g] = fill;
            }
        }
        const uint32_t m = __ballot_sync(0xffffffffu, any);
        if (lane == 0) p.masks[c] = m;
        n_act += __popc(m);
    }
    if (!p.list) {                                                  // masks only: the consumers rank the rows themselves
        if (p.total) {                                              // statistics: one atomic per CTA
            if (lane == 0) s_warp_sums[tid >> 5] = n_act;
            __syncthreads();
            if (tid == 0) {
                int t = 0;
                for (int w = 0; w < COMPACT_THREADS / 32; w++) t += s_warp_sums[w];
                if (t) atomicAdd(p.total, (unsigned long long)t);
            }
        }
        return;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int t = atomicAdd(p.ticket, 1u);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- phase B: this CTA saw every other CTA's masks
    const int per = (n_chunks + COMPACT_THREADS - 1) / COMPACT_THREADS;
    const int c0 = min(tid * per, n_chunks), c1 = min(c0 + per, n_chunks);
    int mine = 0;
    for (int c = c0; c < c1; c++) mine += __popc(__ldcg(p.masks + c));
    int incl = mine;                                   // inclusive scan inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp_sums[tid >> 5] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < (tid >> 5); w++) base += s_warp_sums[w];
    int off = base + incl - mine;
    for (int c = c0; c < c1; c++) {
        uint32_t m = __ldcg(p.masks + c);
        while (m) {
            const int bit = __ffs(m) - 1;
            m &= m - 1;
            p.list[off++] = c * 32 + bit;
        }
    }
    if (tid == COMPACT_THREADS - 1) {
        *p.count = base + incl; *p.ticket = 0u;
        if (p.total) *p.total += (unsigned long long)(base + incl);      // only this thread of this CTA ever writes it
    }
}

int launch_compact(const CompactArgs & a, cudaStream_t st) {
    CompactP p;
    p.idx = a.idx; p.idx_stride = a.idx_stride; p.T = a.T; p.threshold = a.threshold;
    p.n_local = (int)a.n_local; p.bucket = a.bucket; p.list = a.list; p.count = a.count;
    p.masks = a.masks; p.ticket = a.ticket;
    p.zero_dst = a.zero_dst; p.zero_stride = a.zero_stride; p.fill_bias = a.fill_bias; p.fill_relu = a.fill_relu; p.total = a.total;
    const int n_chunks = (int)((a.n_local + 31) / 32);
    int grid = (n_chunks + COMPACT_THREADS / 32 - 1) / (COMPACT_THREADS / 32);
    grid = max(1, min(grid, sm_count()));
    PI_CUDA(launch_k(k_compact, dim3(grid), dim3(COMPACT_THREADS), 0, st, a.pdl, p));
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// axpy, FP16 rows (ggml.c:14314-14463).  CTA = 128 threads x 8 columns = a 1024-column tile; blockIdx.y selects a
// row group: group j takes list entries j, j+G, j+2G, ... in increasing order and keeps the running sums in
// registers, AXPY_UNROLL rows (= 128-bit loads per thread) in flight.  Each group writes one partial vector; the
// partials are summed in group order by the consumer, so the result does not depend on scheduling.
static constexpr int AXPY_F16_THREADS = 128;
static constexpr int AXPY_UNROLL = 4;

struct AxpyP {
    const uint8_t * Wt; int64_t row_bytes; int nrows; int ncols; int nb;
    const float * h; int64_t h_stride;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; int64_t idx_stride; float threshold;
    const int8_t * cq; const float * cd; int64_t c_stride;
    float * partial; int T;
};

template <int TT>
__global__ void __launch_bounds__(AXPY_F16_THREADS) k_axpy_f16(const AxpyP p) {
    const int c = (blockIdx.x * AXPY_F16_THREADS + threadIdx.x) * 8;
    const bool col_ok = c < p.ncols;
    const int G = gridDim.y;
    const int n = min(*p.count, p.nrows);
    float acc[TT][8];
#pragma unroll
    for (int t = 0; t < TT; t++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[t][j] = 0.f;

    for (int i0 = blockIdx.y; i0 < n; i0 += G * AXPY_UNROLL) {
        uint4 w[AXPY_UNROLL];
        float a[AXPY_UNROLL][TT];
#pragma unroll
        for (int u = 0; u < AXPY_UNROLL; u++) {
            const int i = i0 + u * G;
#pragma unroll
            for (int t = 0; t < TT; t++) a[u][t] = 0.f;
            w[u] = make_uint4(0u, 0u, 0u, 0u);
            if (i < n) {
                const int r = p.list[i];
                if ((unsigned)r < (unsigned)p.nrows) {
                    const int64_t g = p.bucket ? p.bucket[r] : r;
                    if (col_ok) w[u] = ldg_stream(p.Wt + (size_t)r * p.row_bytes + (size_t)c * 2);
#pragma unroll
                    for (int t = 0; t < TT; t++) {
                        // the CPU path rounds h to FP16 and skips rows below the threshold (ggml.c:14422-14428)
                        const float hv = round_f16(p.h[(size_t)t * p.h_stride + g]);
                        const bool on = !(p.idx[(size_t)t * p.idx_stride + g] < p.threshold);
                        a[u][t] = on ? hv : 0.f;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < AXPY_UNROLL; u++) {
            const float2 w0 = h2f(w[u].x), w1 = h2f(w[u].y), w2 = h2f(w[u].z), w3 = h2f(w[u].w);
#pragma unroll
            for (int t = 0; t < TT; t++) {
                const float s = a[u][t];
                acc[t][0] = fmaf(w0.x, s, acc[t][0]); acc[t][1] = fmaf(w0.y, s, acc[t][1]);
                acc[t][2] = fmaf(w1.x, s, acc[t][2]); acc[t][3] = fmaf(w1.y, s, acc[t][3]);
                acc[t][4] = fmaf(w2.x, s, acc[t][4]); acc[t][5] = fmaf(w2.y, s, acc[t][5]);
                acc[t][6] = fmaf(w3.x, s, acc[t][6]); acc[t][7] = fmaf(w3.y, s, acc[t][7]);
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int t = 0; t < TT; t++) {
            float * o = p.partial + ((size_t)blockIdx.y * p.T + t) * p.ncols + c;
            *reinterpret_cast<float4 *>(o)     = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
            *reinterpret_cast<float4 *>(o + 4) = make_float4(acc[t][4], acc[t][5], acc[t][6], acc[t][7]);
        }
    }
}

// axpy, planar Q4_0 rows (ggml.c:14465-14618, ggml-quants.c:2426-2509).  One thread per 32-column block of the row:
// a 128-bit load brings the block's nibbles, the thread keeps 32 running sums.  The neuron's coefficient is the int8
// quant b of h over its 32-NEURON block times that block's FP16 scale d8; (q-8) is rebuilt as an exact float by
// splicing the nibble into the mantissa of 2^23 and subtracting 2^23+8, so no int->float conversion is issued.
static constexpr int AXPY_Q4_THREADS = 128;

__device__ __forceinline__ float nib_to_float(uint32_t bytes, int k) {      // byte k of `bytes` holds 0..15
    const uint32_t sel = 0x7650u | (uint32_t)k;                                 // {b3,b2,b1,b0} = {0x4B,0x00,0x00,byte k}
    const uint32_t bits = __byte_perm(bytes, 0x4B000000u, sel);
    return __uint_as_float(bits) - 8388616.0f;
}

template <int TT>
__global__ void __launch_bounds__(AXPY_Q4_THREADS) k_axpy_q4(const AxpyP p) {
    const int b = blockIdx.x * AXPY_Q4_THREADS + threadIdx.x;
    const bool col_ok = b < p.nb;
    const int G = gridDim.y;
    const int n = min(*p.count, p.nrows);
    float acc[TT][32];
#pragma unroll
    for (int t = 0; t < TT; t++)
#pragma unroll
        for (int j = 0; j < 32; j++) acc[t][j] = 0.f;

    for (int i0 = blockIdx.y; i0 < n; i0 += G * AXPY_UNROLL) {
        uint4 q[AXPY_UNROLL];
        float s[AXPY_UNROLL][TT];
#pragma unroll
        for (int u = 0; u < AXPY_UNROLL; u++) {
            const int i = i0 + u * G;
#pragma unroll
            for (int t = 0; t < TT; t++) s[u][t] = 0.f;
            q[u] = make_uint4(0u, 0u, 0u, 0u);
            if (i < n) {
                const int r = p.list[i];
                if ((unsigned)r < (unsigned)p.nrows && col_ok) {
                    const int64_t g = p.bucket ? p.bucket[r] : r;
                    const uint8_t * row = p.Wt + (size_t)r * p.row_bytes;
                    q[u] = ldg_stream(reinterpret_cast<const uint4 *>(row) + b);
                    const float d4 = __half2float(__ldg(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16) + b));
#pragma unroll
                    for (int t = 0; t < TT; t++) {
                        const bool on = !(p.idx[(size_t)t * p.idx_stride + g] < p.threshold);
                        const int b8 = p.cq[(size_t)t * p.c_stride + g];
                        const float d8 = p.cd[(size_t)t * (p.c_stride / QK) + g / QK];
                        s[u][t] = on ? (float)b8 * (d4 * d8) : 0.f;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < AXPY_UNROLL; u++) {
            const uint32_t wds[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const uint32_t lo = wds[wi] & 0x0F0F0F0Fu, hi = (wds[wi] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float vlo = nib_to_float(lo, k), vhi = nib_to_float(hi, k);
#pragma unroll
                    for (int t = 0; t < TT; t++) {
                        acc[t][wi * 4 + k]      = fmaf(vlo, s[u][t], acc[t][wi * 4 + k]);
                        acc[t][16 + wi * 4 + k] = fmaf(vhi, s[u][t], acc[t][16 + wi * 4 + k]);
                    }
                }
            }
        }
    }
    if (col_ok) {
#pragma unroll
        for (int t = 0; t < TT; t++) {
            float * o = p.partial + ((size_t)blockIdx.y * p.T + t) * p.ncols + (size_t)b * QK;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4 *>(o + j) = make_float4(acc[t][j], acc[t][j + 1], acc[t][j + 2], acc[t][j + 3]);
        }
    }
}

// Row groups: enough CTAs to keep ~6 resident per SM (each holds AXPY_UNROLL x 2 KB of loads in flight), capped
// so the partial buffer stays small next to the weight bytes.
int axpy_groups(int wtype, int64_t ncols, int T) {
    (void)T;      // the buffer must fit the largest group count of any kernel the launcher may pick
    const int tiles = wtype == PI_TYPE_Q4_0 ? (int)((ncols / QK + AXPY_Q4_THREADS - 1) / AXPY_Q4_THREADS)
                                            : (int)((ncols / 8 + AXPY_F16_THREADS - 1) / AXPY_F16_THREADS);
    int g = (sm_count() * 6 + tiles - 1) / tiles;
    return max(sm_count(), min(g, 256));
}

int launch_axpy(const AxpyArgs & a, cudaStream_t st, int * groups_used) {
    if (a.T <= 0) return PI_OK;
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    if (groups_used) *groups_used = a.n_groups;
    if (a.T == 1 && a.masks) {                                      // one token, rows named by bit masks
        const int rc = launch_axpy_rows(a, st, groups_used);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
        if (!a.list) { set_error("axpy: masks given but the shape is not eligible and there is no list"); return PI_ERR_UNSUPPORTED; }
        if (groups_used) *groups_used = a.n_groups;
    }
    if (a.T > 1 && a.status) {                                      // 2..32 tokens: tensor-core kernels
        const int rc = launch_axpy_mma(a, st, groups_used);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
        if (groups_used) *groups_used = a.n_groups;
    }
    // CUDA-core kernels for what the kernels above decline.  Q4_0 rows read the coefficient planes (int8 quant of h per
    // 32 neurons, block scale); callers fill them for batches, a single token gets them here.
    if (q4 && a.T == 1) {
        PI_REQUIRE(a.cq && a.cd, "axpy: Q4_0 needs coefficient planes");
        const int rc = launch_neuron_q8(a.h, a.h_stride, a.h_stride, 1, const_cast<int8_t *>(a.cq), const_cast<float *>(a.cd), st);
        if (rc) return rc;
    }
    AxpyP p;
    p.Wt = (const uint8_t *)a.Wt; p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols);
    p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK);
    p.h_stride = a.h_stride; p.list = a.list; p.count = a.count; p.bucket = a.bucket;
    p.idx_stride = a.idx_stride; p.threshold = a.threshold; p.c_stride = a.c_stride; p.T = a.T;
    const int tiles = q4 ? (p.nb + AXPY_Q4_THREADS - 1) / AXPY_Q4_THREADS : (p.ncols / 8 + AXPY_F16_THREADS - 1) / AXPY_F16_THREADS;
    const dim3 grid(tiles, a.n_groups);
    const int max_tt = q4 ? 2 : 4;                                      // register budget: 32 (8) sums per token
    for (int t0 = 0; t0 < a.T; ) {
        const int left = a.T - t0;
        int tt = 1;
        while (tt * 2 <= left && tt * 2 <= max_tt) tt *= 2;
        p.h = a.h ? a.h + (size_t)t0 * a.h_stride : nullptr;
        p.idx = a.idx + (size_t)t0 * a.idx_stride;
        p.cq = a.cq ? a.cq + (size_t)t0 * a.c_stride : nullptr;
        p.cd = a.cd ? a.cd + (size_t)t0 * (a.c_stride / QK) : nullptr;
        p.partial = a.partial + (size_t)t0 * a.ncols;                   // token t of group j lives at [j, t, :]
        if (q4) {
            if (tt == 2) k_axpy_q4<2><<<grid, AXPY_Q4_THREADS, 0, st>>>(p);
            else         k_axpy_q4<1><<<grid, AXPY_Q4_THREADS, 0, st>>>(p);
        } else {
            if (tt == 4)      k_axpy_f16<4><<<grid, AXPY_F16_THREADS, 0, st>>>(p);
            else if (tt == 2) k_axpy_f16<2><<<grid, AXPY_F16_THREADS, 0, st>>>(p);
            else              k_axpy_f16<1><<<grid, AXPY_F16_THREADS, 0, st>>>(p);
        }
        PI_LAUNCH_CHECK("k_axpy");
        t0 += tt;
    }
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// dst[t, c] = sum_j partial[j, t, c] (j ascending within each of 32 interleaved classes, classes added in order)
//             + bias[c] + residual[t, c].  A CTA owns 128 consecutive values; warp w adds groups w, w+32, w+64, ...;
// the 32 warp sums are then added in warp order.  The order is fixed, so the result is reproducible.
static constexpr int RED_WARPS = 32;

__global__ void __launch_bounds__(RED_WARPS * 32) k_reduce_partials(const float * __restrict__ partial, int G, int64_t total, int64_t n,
                                                                     const float * __restrict__ residual, const float * __restrict__ bias,
                                                                     float * __restrict__ dst, const float * __restrict__ residual2,
                                                                     double * __restrict__ stats_out) {
    __shared__ float4 s_part[RED_WARPS][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    pdl_launch();
    pdl_wait();
    const int64_t i4 = (int64_t)blockIdx.x * 32 + lane;                // float4 index
    const bool ok = i4 * 4 < total;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
        for (int j0 = w; j0 < G; j0 += RED_WARPS * 8) {                // 8 loads in flight, added in group order
            float4 a[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int j = j0 + u * RED_WARPS;
                a[u] = j < G ? __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)j * total) + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
        }
    }
    s_part[w][lane] = v;
    __syncthreads();
    if (w == 0 && ok) {
#pragma unroll
        for (int k = 1; k < RED_WARPS; k++) { const float4 a = s_part[k][lane]; v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
        const int64_t i = i4 * 4;
        if (bias) { const int64_t c = i % n; v.x += bias[c]; v.y += bias[c + 1]; v.z += bias[c + 2]; v.w += bias[c + 3]; }
        if (residual2) { const float4 r = *reinterpret_cast<const float4 *>(residual2 + i); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
        if (residual) { const float4 r = *reinterpret_cast<const float4 *>(residual + i); v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; }
        *reinterpret_cast<float4 *>(dst + i) = v;
    }
    if (w == 0 && stats_out) {                                         // the next norm's statistics ride along (T == 1)
        double s1 = ok ? (double)v.x + (double)v.y + (double)v.z + (double)v.w : 0.0;
        double s2 = ok ? (double)(v.x * v.x) + (double)(v.y * v.y) + (double)(v.z * v.z) + (double)(v.w * v.w) : 0.0;
        s1 = warp_sum_d(s1); s2 = warp_sum_d(s2);
        if (lane == 0) { atomicAdd(stats_out, s1); atomicAdd(stats_out + 1, s2); }
    }
}

int launch_reduce_partials(const float * partial, int n_groups, int T, int64_t n, const float * residual,
                           const float * bias, float * dst, cudaStream_t st, bool pdl, const float * residual2, double * stats_out) {
    const int64_t total = (int64_t)T * n;
    if (total == 0) return PI_OK;
    PI_REQUIRE(n % 4 == 0, "reduce: n must be a multiple of 4");
    const int grid = (int)((total / 4 + 31) / 32);
    PI_CUDA(launch_k(k_reduce_partials, dim3(grid), dim3(RED_WARPS * 32), 0, st, pdl, partial, n_groups, total, n, residual, bias, dst, residual2, stats_out));
    return PI_OK;
}

}  // namespace pi
