// The neuron-sparse half of the FFN: predictor mask -> compacted active list (warp ballot / popc), and the
// scatter-accumulate behind ggml_axpy over the rows of ffn_down_t named by that list.
#include "pi_common.cuh"

#include <cstdlib>

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
    int32_t * parts; int n_parts; int32_t * chunk_off;
};

__global__ void __launch_bounds__(COMPACT_THREADS) k_compact(const CompactP p) {
    __shared__ int s_last;
    __shared__ int s_warp_sums[COMPACT_THREADS / 32];
    const int tid = threadIdx.x, lane = tid & 31;
    const int n_chunks = (p.n_local + 31) / 32;
    const int warps_total = gridDim.x * (COMPACT_THREADS / 32);
    pdl_launch();
    pdl_wait();
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
    if (p.parts) {                                                  // exclusive prefix per 32-row chunk, for the balanced split below
        int o = off;
        for (int c = c0; c < c1; c++) { p.chunk_off[c] = o; o += __popc(__ldcg(p.masks + c)); }
        if (tid == COMPACT_THREADS - 1) p.chunk_off[n_chunks] = base + incl;
    }
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
    if (p.parts) {
        // Split the chunks into n_parts contiguous ranges of (nearly) equal active-row count: part j starts at the first
        // chunk whose exclusive prefix reaches j * total / n_parts.  Whole chunks (32 consecutive neurons) stay together,
        // which is what the Q4_0 axpy coefficient (quantised per 32 neurons) needs.
        __shared__ int s_total;
        if (tid == COMPACT_THREADS - 1) s_total = base + incl;
        __threadfence_block();
        __syncthreads();
        const int total = s_total;
        for (int j = tid; j <= p.n_parts; j += COMPACT_THREADS) {
            int lo = 0, hi = n_chunks;                                  // lower_bound over chunk_off[0..n_chunks]
            if (j == p.n_parts) { lo = n_chunks; }
            else if (j > 0) {
                const int target = (int)(((long long)j * total + p.n_parts - 1) / p.n_parts);
                while (lo < hi) {
                    const int mid = (lo + hi) >> 1;
                    if (p.chunk_off[mid] >= target) hi = mid; else lo = mid + 1;
                }
            }
            p.parts[j] = lo;
        }
    }
}

int launch_compact(const CompactArgs & a, cudaStream_t st) {
    CompactP p;
    p.idx = a.idx; p.idx_stride = a.idx_stride; p.T = a.T; p.threshold = a.threshold;
    p.n_local = (int)a.n_local; p.bucket = a.bucket; p.list = a.list; p.count = a.count;
    p.masks = a.masks; p.ticket = a.ticket;
    p.zero_dst = a.zero_dst; p.zero_stride = a.zero_stride; p.fill_bias = a.fill_bias; p.fill_relu = a.fill_relu; p.total = a.total;
    p.parts = a.parts; p.n_parts = a.n_parts; p.chunk_off = a.chunk_off;
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

// ------------------------------------------------------------------------------------------------
// axpy for one token, bulk-copy pipelined (the batch-1 decode path).  One persistent CTA per SM walks list entries
// cta, cta+G, cta+2G, ... in increasing order.  Whole weight rows (contiguous in both layouts: FP16, or planar Q4_0 =
// nibbles then scales) are staged in shared memory by the bulk-copy engine (cp.async.bulk, non-tensor, no multicast)
// into a ring of PIPE stages, each guarded by an mbarrier that counts the row's bytes, so a CTA keeps 100+ KB of
// loads in flight without holding them in registers.  Threads own fixed columns and keep their sums in registers;
// the per-CTA partial vectors are summed in CTA order afterwards (no atomics, fixed order).
// The coefficient of each row is made in the prologue with the CPU path's rule: FP16(h) for FP16 rows; for Q4_0 the
// int8 quant of h within its block of 32 neurons times that block's FP16 scale (ggml.c:14575-14581).
// Every mbarrier wait is bounded; if one runs out the CTA raises bit 1 of *status, stops consuming and still writes
// its partial, so a lost copy can never hang the GPU.
static constexpr int PIPE_MAX_ROWS = 512;               // list entries one CTA may own (F / G, rounded up)

struct AxpyPipeP {
    const uint8_t * Wt; int64_t row_bytes; int nrows; int ncols; int nb;
    const float * h; const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; float threshold;
    float * partial; unsigned int * status; int stages; int max_rows;
};

static constexpr int PIPE_RS = 4;                       // rows per ring stage (one barrier, one CTA-wide sync per stage)

// Up to 1024 threads per CTA so that 32 warps hide the shared-memory and ALU latencies.  FP16: a thread owns CPT chunks of
// 8 columns (chunk = tid + k * blockDim).  Q4_0: a thread owns ONE 32-bit word of a block's nibbles = 8 columns
// (4 low-nibble columns 4i.., 4 high-nibble columns 16+4i..), four threads share a block's scale.
template <int WT, int CPT>
__global__ void __launch_bounds__(1024) k_axpy_pipe(const AxpyPipeP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nwarp = blockDim.x >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages;
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);                      // [S]
    int *   rows = reinterpret_cast<int *>(smem + 8 * 32);                     // [max_rows]
    float * coef = reinterpret_cast<float *>(rows + p.max_rows);               // [max_rows]
    unsigned char * ring = smem + (((size_t)8 * 32 + (size_t)8 * p.max_rows + 127) & ~(size_t)127);
    const size_t row_stride = ((size_t)p.row_bytes + 127) & ~(size_t)127;
    const size_t stage_bytes = row_stride * PIPE_RS;

    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    pdl_launch();
    pdl_wait();
    // the list entry this thread would own is read together with the count, not after it (the list buffer has nrows
    // entries whatever the count; what lies beyond the count is stale and is dropped below): one round trip, not two
    int spec = -1;
    if (tid < p.max_rows && cta + tid * G < p.nrows) spec = p.list[cta + tid * G];
    const int n = min(*p.count, p.nrows);
    int n_mine = cta < n ? (n - cta + G - 1) / G : 0;
    n_mine = min(n_mine, p.max_rows);
    const int n_stages = (n_mine + PIPE_RS - 1) / PIPE_RS;

    // ---- prologue: my rows first, start the copies, then the coefficients while the rows fly in
    for (int i = tid; i < n_mine; i += blockDim.x) {
        const int r = i == tid ? spec : p.list[cta + i * G];
        rows[i] = (unsigned)r < (unsigned)p.nrows ? r : -1;
    }
    __syncthreads();
    auto issue = [&](int st) {                                       // all lanes of warp 0
        const int s = st % S;
        const int cnt = min(PIPE_RS, n_mine - st * PIPE_RS);
        // the phase cannot complete before this arrive, whatever the order in which the lanes' copies land
        if (lane == 0) mbar_expect_tx(full + s, (unsigned)(cnt * p.row_bytes));
        if (lane < cnt) {
            const int r = rows[st * PIPE_RS + lane] < 0 ? 0 : rows[st * PIPE_RS + lane];
            bulk_g2s(ring + s * stage_bytes + lane * row_stride, p.Wt + (size_t)r * p.row_bytes, (unsigned)p.row_bytes, full + s);
        }
    };
    PI_TL_MARK(0);
    if (wid == 0) for (int st = 0; st < S && st < n_stages; st++) issue(st);
    PI_TL_MARK(1);
    // warp 0 is busy issuing the copies (~80 ns each): the coefficients are the other warps' work
    const int cw = nwarp > 1 ? nwarp - 1 : 1, cw0 = nwarp > 1 ? wid - 1 : 0;
    for (int i0 = cw0; i0 >= 0 && i0 < n_mine; i0 += cw * 4) {     // 4 rows per warp per pass: their loads overlap
        float hv[4], pv[4]; int64_t g[4]; bool ok[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * cw;
            ok[u] = i < n_mine && rows[i] >= 0;
            const int r = ok[u] ? rows[i] : 0;
            g[u] = p.bucket ? p.bucket[r] : r;
            hv[u] = WT == PI_TYPE_F16 ? p.h[g[u]] : p.h[(g[u] & ~(int64_t)31) + lane];
            pv[u] = p.idx[g[u]];
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * cw;
            float c;
            if (WT == PI_TYPE_F16) {
                c = round_f16(hv[u]);
            } else {
                const float amax = warp_max(fabsf(hv[u]));
                const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
                const int q = __float2int_rn(hv[u] * id);
                const int b8 = __shfl_sync(0xffffffffu, q, (int)(g[u] & 31));
                c = (float)b8 * round_f16(amax / 127.0f);
            }
            if (!ok[u] || pv[u] < p.threshold) c = 0.f;
            if (lane == 0 && i < n_mine) coef[i] = c;
        }
    }
    __syncthreads();

    PI_TL_MARK(2);
    constexpr int NACC = WT == PI_TYPE_F16 ? CPT * 8 : 8;
    float acc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; j++) acc[j] = 0.f;
    const int n_chunks = p.ncols / 8;
    const int n_words = p.nb * 4;
    bool dead = false;                                               // warp-uniform
    float corr = 0.f;                                                // Q4_0: sum of the row scales (see the dequantisation below)

    for (int st = 0; st < n_stages; st++) {
        const int s = st % S;
        const unsigned parity = (unsigned)(st / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) {
                if (++spins > (1 << 20)) { gave_up = true; break; }    // each try_wait already blocks for a while
            }
            dead = __any_sync(0xffffffffu, gave_up) != 0;
            if (dead && lane == 0) atomicOr(p.status, 2u);
        }
        if (st == 0) PI_TL_MARK(3);
        const int cnt = min(PIPE_RS, n_mine - st * PIPE_RS);
        if (!dead) {
#pragma unroll
            for (int k = 0; k < PIPE_RS; k++) {
                if (k >= cnt) break;
                const float c = coef[st * PIPE_RS + k];
                if (c == 0.f) continue;
                const unsigned char * row = ring + s * stage_bytes + k * row_stride;
                if (WT == PI_TYPE_F16) {
#pragma unroll
                    for (int q = 0; q < CPT; q++) {
                        const int ch = tid + q * (int)blockDim.x;
                        if (ch < n_chunks) {
                            const uint4 w = reinterpret_cast<const uint4 *>(row)[ch];
                            const float2 w0 = h2f(w.x), w1 = h2f(w.y), w2 = h2f(w.z), w3 = h2f(w.w);
                            acc[q * 8 + 0] = fmaf(w0.x, c, acc[q * 8 + 0]); acc[q * 8 + 1] = fmaf(w0.y, c, acc[q * 8 + 1]);
                            acc[q * 8 + 2] = fmaf(w1.x, c, acc[q * 8 + 2]); acc[q * 8 + 3] = fmaf(w1.y, c, acc[q * 8 + 3]);
                            acc[q * 8 + 4] = fmaf(w2.x, c, acc[q * 8 + 4]); acc[q * 8 + 5] = fmaf(w2.y, c, acc[q * 8 + 5]);
                            acc[q * 8 + 6] = fmaf(w3.x, c, acc[q * 8 + 6]); acc[q * 8 + 7] = fmaf(w3.y, c, acc[q * 8 + 7]);
                        }
                    }
                } else if (tid < n_words) {
                    const uint32_t word = reinterpret_cast<const uint32_t *>(row)[tid];
                    // nibble q -> the float 0.5 + q/256 with one byte permute (q lands in mantissa bits 16..19 under the
                    // exponent of 0.5); (q - 8) * sc = (0.5 + q/256) * 256 sc - 0.53125 * 256 sc, and the second term is
                    // summed once per row instead of once per weight.  Costs ~4 bits of the FP32 accumulator.
                    const float sc = 256.0f * c * __half2float(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16)[tid >> 2]);
                    const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;
                    corr += sc;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        acc[j]     = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044u | (uint32_t)(j << 8))), sc, acc[j]);
                        acc[4 + j] = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044u | (uint32_t)(j << 8))), sc, acc[4 + j]);
                    }
                }
            }
        }
        if (st + S < n_stages) {                                     // block-uniform: the stage is reused, so everyone must be done with it
            __syncthreads();
            if (wid == 0 && !dead) issue(st + S);
        }
    }
    // a CTA that gave up must not leave copies in flight into its shared memory: drain what was issued
    if (__syncthreads_or(dead) && tid == 0) {
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }

    PI_TL_MARK(4);
    float * out = p.partial + (size_t)cta * p.ncols;
    if (WT == PI_TYPE_F16) {
#pragma unroll
        for (int q = 0; q < CPT; q++) {
            const int ch = tid + q * (int)blockDim.x;
            if (ch < n_chunks) {
                *reinterpret_cast<float4 *>(out + ch * 8)     = make_float4(acc[q * 8 + 0], acc[q * 8 + 1], acc[q * 8 + 2], acc[q * 8 + 3]);
                *reinterpret_cast<float4 *>(out + ch * 8 + 4) = make_float4(acc[q * 8 + 4], acc[q * 8 + 5], acc[q * 8 + 6], acc[q * 8 + 7]);
            }
        }
    } else if (tid < n_words) {
        const int b = tid >> 2, i = tid & 3;
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = fmaf(-0.53125f, corr, acc[j]);
        *reinterpret_cast<float4 *>(out + (size_t)b * QK + 4 * i)      = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4 *>(out + (size_t)b * QK + 16 + 4 * i) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

struct PipePlan { bool ok; int threads; int cpt; int stages; int max_rows; size_t smem; int groups; };

static PipePlan pipe_plan(int wtype, int64_t nrows, int64_t ncols) {
    PipePlan pl{};
    const int G = sm_count();
    const size_t row_bytes = pi_row_bytes(wtype, ncols);
    const size_t row_stride = (row_bytes + 127) & ~size_t(127);
    pl.groups = G;
    pl.max_rows = (int)((nrows + G - 1) / G);
    if (pl.max_rows > PIPE_MAX_ROWS || row_bytes % 16 != 0) return pl;
    if (wtype == PI_TYPE_Q4_0) {
        const int nb = (int)(ncols / QK);
        if (nb * 4 > 1024) return pl;
        pl.threads = (nb * 4 + 31) / 32 * 32; pl.cpt = 1;
    } else {
        const int chunks = (int)(ncols / 8);
        pl.threads = chunks >= 1024 ? 1024 : (chunks + 31) / 32 * 32;
        pl.cpt = (chunks + pl.threads - 1) / pl.threads;
        if (pl.cpt > 2) return pl;
    }
    const size_t head = ((size_t)8 * 32 + (size_t)8 * pl.max_rows + 127 + 128) & ~size_t(127);
    static size_t budget = 0;
    if (!budget) { const char * v = getenv("PI_AXPY_KB"); budget = (size_t)(v ? atoi(v) : 200) * 1024; }
    int S = (int)((budget - head) / (row_stride * PIPE_RS));
    S = S > 16 ? 16 : S;
    if (S < 2) return pl;
    pl.stages = S;
    pl.smem = head + (size_t)S * row_stride * PIPE_RS;
    pl.ok = true;
    return pl;
}

template <int WT, int CPT>
static int launch_pipe_inst(const AxpyPipeP & p, const PipePlan & pl, cudaStream_t st, bool pdl) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_axpy_pipe<WT, CPT>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(pl.groups), dim3(pl.threads), pl.smem, st, pdl, p));
    return PI_OK;
}

// Row groups: enough CTAs to keep ~6 resident per SM (each holds AXPY_UNROLL x 2 KB of loads in flight), capped
// so the partial buffer stays small next to the weight bytes.
int axpy_groups(int wtype, int64_t ncols, int T) {
    (void)T;      // the buffer must fit the larger of the two kernels' group counts: the pipelined one uses one CTA per SM
    const int tiles = wtype == PI_TYPE_Q4_0 ? (int)((ncols / QK + AXPY_Q4_THREADS - 1) / AXPY_Q4_THREADS)
                                            : (int)((ncols / 8 + AXPY_F16_THREADS - 1) / AXPY_F16_THREADS);
    int g = (sm_count() * 6 + tiles - 1) / tiles;
    return max(sm_count(), min(g, 256));
}

int launch_axpy(const AxpyArgs & a, cudaStream_t st, int * groups_used) {
    if (a.T <= 0) return PI_OK;
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    if (groups_used) *groups_used = a.n_groups;
    if (a.T > 1 && a.status) {                                      // 2..32 tokens: tensor-core kernels
        const int rc = launch_axpy_mma(a, st, groups_used);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
        if (groups_used) *groups_used = a.n_groups;
    }
    if (a.T == 1 && a.status) {
        const PipePlan pl = pipe_plan(a.wtype, a.nrows, a.ncols);
        if (pl.ok && pl.groups <= a.n_groups) {
            AxpyPipeP p;
            p.Wt = (const uint8_t *)a.Wt; p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols); p.nrows = (int)a.nrows;
            p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK);
            p.h = a.h; p.list = a.list; p.count = a.count; p.bucket = a.bucket; p.idx = a.idx; p.threshold = a.threshold;
            p.partial = a.partial; p.status = a.status; p.stages = pl.stages; p.max_rows = pl.max_rows;
            if (groups_used) *groups_used = pl.groups;
            if (q4) return launch_pipe_inst<PI_TYPE_Q4_0, 1>(p, pl, st, a.pdl);
            if (pl.cpt == 1) return launch_pipe_inst<PI_TYPE_F16, 1>(p, pl, st, a.pdl);
            return launch_pipe_inst<PI_TYPE_F16, 2>(p, pl, st, a.pdl);
        }
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
