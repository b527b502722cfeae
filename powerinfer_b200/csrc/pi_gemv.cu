// Warp-per-row mat-vec over FP16 and planar-Q4_0 weight rows: the dense decode mat-vecs (predictor, QKV, out-proj,
// lm head) and the gather mat-vec behind ggml_mul_mat_idx, which walks a compacted list of active rows.
//
// HBM-bound: every weight byte is read once with 128-bit streaming loads (L1 no-allocate), UNROLL loads in flight
// per lane; the activation (FP16, or Q8_0 planes) is staged once per CTA in shared memory and reused by all rows the
// CTA visits.  Rows are handed to warps round-robin from a persistent grid of (SMs x resident CTAs), so the launch
// shape never depends on the number of active rows (it is read from device memory), which keeps the kernel
// capturable in a CUDA graph.
#include "pi_common.cuh"

namespace pi {

static constexpr int QK = 32;
static constexpr int GEMV_THREADS = 256;
static constexpr int GEMV_WARPS = GEMV_THREADS / 32;
static constexpr int LOADS = 16;          // 128-bit weight loads one lane keeps in flight (split over the rows it works on)

struct GemvP {
    const uint8_t * W; const uint8_t * W2;
    int64_t row_bytes; int nrows; int ncols; int nb;
    Act x; int T;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; int64_t idx_stride; float threshold;
    const float * bias; int relu;
    float * dst; __half * dst16; int64_t dst_stride;
};

struct SmemQ8 {            // staged Q8_0 planes of TT tokens
    const uint4 * lo; const uint4 * hi; const float * d; const int * s;
};

// Integer dot of one Q4_0 block (16 bytes of nibbles) with one Q8_0 block held as two planes (values 0..15, 16..31).
// Nibbles are taken as 0..15 and the offset of 8 is removed with the block's int8 sum: sum((q-8) x) = sum(q x) - 8 sum(x).
__device__ __forceinline__ int block_dot_q4_q8(const uint4 q, const uint4 lo, const uint4 hi, int s8) {
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

// Dots of NR weight rows (same column range [c_lo, c_hi) of each) with TT staged activation vectors.  All NR x U loads of
// a column batch are issued before any of them is consumed.  FP16: a lane owns 8 consecutive columns per 256-column
// step.  rows[i] == nullptr skips row i.
template <int TT, int NR>
__device__ __forceinline__ void rows_dot_f16(const uint8_t * const (&rows)[NR], int c_lo, int c_hi, int ncols,
                                             const __half * __restrict__ xs, int lane, float (&acc)[NR][TT]) {
    constexpr int U = LOADS / NR;
    for (int c0 = c_lo + lane * 8; c0 < c_hi; c0 += 256 * U) {
        uint4 w[NR][U];
#pragma unroll
        for (int r = 0; r < NR; r++)
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int c = c0 + u * 256;
                if (rows[r] && c < c_hi) w[r][u] = ldg_stream(rows[r] + (size_t)c * 2);
            }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int c = c0 + u * 256;
            if (c < c_hi) {
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    const uint4 xv = *reinterpret_cast<const uint4 *>(xs + (size_t)t * ncols + c);
                    const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        if (!rows[r]) continue;
                        const float2 w0 = h2f(w[r][u].x), w1 = h2f(w[r][u].y), w2 = h2f(w[r][u].z), w3 = h2f(w[r][u].w);
                        float a = acc[r][t];
                        a = fmaf(w0.x, x0.x, a); a = fmaf(w0.y, x0.y, a);
                        a = fmaf(w1.x, x1.x, a); a = fmaf(w1.y, x1.y, a);
                        a = fmaf(w2.x, x2.x, a); a = fmaf(w2.y, x2.y, a);
                        a = fmaf(w3.x, x3.x, a); a = fmaf(w3.y, x3.y, a);
                        acc[r][t] = a;
                    }
                }
            }
        }
    }
}

// planar Q4_0: a lane owns one 32-column block per 32-block step; [b_lo, b_hi) is the block range
template <int TT, int NR>
__device__ __forceinline__ void rows_dot_q4(const uint8_t * const (&rows)[NR], int b_lo, int b_hi, int nb, const SmemQ8 xs,
                                            int lane, float (&acc)[NR][TT]) {
    constexpr int U = LOADS / NR;
    for (int b0 = b_lo + lane; b0 < b_hi; b0 += 32 * U) {
        uint4 q[NR][U];
        __half sc[NR][U];
#pragma unroll
        for (int r = 0; r < NR; r++)
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int b = b0 + u * 32;
                if (rows[r] && b < b_hi) {
                    q[r][u] = ldg_stream(reinterpret_cast<const uint4 *>(rows[r]) + b);
                    sc[r][u] = __ldg(reinterpret_cast<const __half *>(rows[r] + (size_t)nb * 16) + b);
                }
            }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int b = b0 + u * 32;
            if (b < b_hi) {
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    const int i = t * nb + b;
                    const uint4 lo = xs.lo[i], hi = xs.hi[i];
                    const int s8 = xs.s[i];
                    const float d8 = xs.d[i];
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        if (!rows[r]) continue;
                        const int sumi = block_dot_q4_q8(q[r][u], lo, hi, s8);
                        acc[r][t] = fmaf((float)sumi, __half2float(sc[r][u]) * d8, acc[r][t]);
                    }
                }
            }
        }
    }
}

// One work item = one row (dense) or one list entry (sparse), optionally split column-wise over SPLIT warps of the same
// CTA.  A warp works on PAIR items at once (and on the gate row of each, when GATED), so NR = PAIR x (GATED ? 2 : 1) rows
// are streamed together.  The CTA-level loop is uniform, so the shared-memory combine of split rows may synchronise.
template <int WT, int TT, bool SPARSE, bool GATED, int SPLIT, int PAIR>
__global__ void __launch_bounds__(GEMV_THREADS) k_gemv(const GemvP p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float s_part[GEMV_WARPS][PAIR * (GATED ? 2 : 1)][TT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch();
    pdl_wait();
    constexpr int NR = PAIR * (GATED ? 2 : 1);
    constexpr int ITEMS_PER_CTA = (GEMV_WARPS / SPLIT) * PAIR;

    // ---- stage the activation of TT tokens
    SmemQ8 xq;
    const __half * xh = reinterpret_cast<const __half *>(smem);
    if (WT == PI_TYPE_F16) {
        const int n16 = (TT * p.ncols * 2) / 16;
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dst = reinterpret_cast<uint4 *>(smem);
        for (int i = tid; i < n16; i += GEMV_THREADS) dst[i] = src[i];
    } else {
        const int n = TT * p.nb;
        uint4 * lo = reinterpret_cast<uint4 *>(smem);
        uint4 * hi = lo + n;
        float * d = reinterpret_cast<float *>(hi + n);
        int * s = reinterpret_cast<int *>(d + n);
        for (int i = tid; i < n; i += GEMV_THREADS) { lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i]; d[i] = p.x.d[i]; s[i] = p.x.s[i]; }
        xq.lo = lo; xq.hi = hi; xq.d = d; xq.s = s;
    }
    __syncthreads();

    const int n_items = SPARSE ? min(*p.count, p.nrows) : p.nrows;
    const int part = warp % SPLIT;
    const int slot = warp / SPLIT;                                  // which of the CTA's concurrent items this warp serves

    for (int base = blockIdx.x * ITEMS_PER_CTA; base < n_items; base += gridDim.x * ITEMS_PER_CTA) {
        int r[PAIR];
        const uint8_t * rows[NR];
        float acc[NR][TT];
#pragma unroll
        for (int k = 0; k < PAIR; k++) {
            const int it = base + slot * PAIR + k;
            int rr = -1;
            if (it < n_items) {
                rr = SPARSE ? p.list[it] : it;
                if ((unsigned)rr >= (unsigned)p.nrows) rr = -1;    // a damaged list must not turn into a wild read
            }
            r[k] = rr;
            rows[k] = rr >= 0 ? p.W + (size_t)rr * p.row_bytes : nullptr;
            if (GATED) rows[PAIR + k] = rr >= 0 ? p.W2 + (size_t)rr * p.row_bytes : nullptr;
        }
#pragma unroll
        for (int i = 0; i < NR; i++)
#pragma unroll
            for (int t = 0; t < TT; t++) acc[i][t] = 0.f;

        if (WT == PI_TYPE_F16) {
            const int per = p.ncols / SPLIT;                          // SPLIT > 1 only when ncols % (256 * SPLIT) == 0
            rows_dot_f16<TT, NR>(rows, part * per, (part + 1) * per, p.ncols, xh, lane, acc);
        } else {
            const int per = p.nb / SPLIT;
            rows_dot_q4<TT, NR>(rows, part * per, (part + 1) * per, p.nb, xq, lane, acc);
        }
#pragma unroll
        for (int i = 0; i < NR; i++)
#pragma unroll
            for (int t = 0; t < TT; t++) acc[i][t] = warp_sum(acc[i][t]);

        if (SPLIT > 1) {
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < NR; i++)
#pragma unroll
                    for (int t = 0; t < TT; t++) s_part[warp][i][t] = acc[i][t];
            }
            __syncthreads();
            if (part == 0) {
#pragma unroll
                for (int i = 0; i < NR; i++)
#pragma unroll
                    for (int t = 0; t < TT; t++) {
                        float v = s_part[warp][i][t];
                        for (int q = 1; q < SPLIT; q++) v += s_part[warp + q][i][t];
                        acc[i][t] = v;
                    }
            }
        }
        if (part == 0) {
#pragma unroll
            for (int k = 0; k < PAIR; k++) {
                if (r[k] < 0) continue;
                const int64_t g = SPARSE && p.bucket ? p.bucket[r[k]] : r[k];
                if (lane < TT) {
                    float v = 0.f, v2 = 0.f;
#pragma unroll
                    for (int t = 0; t < TT; t++) if (lane == t) { v = acc[k][t]; if (GATED) v2 = acc[PAIR + k][t]; }
                    const int t = lane;
                    bool active = true;
                    if (SPARSE) active = !(p.idx[(size_t)t * p.idx_stride + g] < p.threshold);
                    float o = active ? v : 0.f;
                    if (GATED) o = active ? fmaxf(v2, 0.f) * v : 0.f;
                    if (p.bias) o += p.bias[g];
                    if (p.relu) o = fmaxf(o, 0.f);
                    if (p.dst)   p.dst[(size_t)t * p.dst_stride + g] = o;
                    if (p.dst16) p.dst16[(size_t)t * p.dst_stride + g] = __float2half_rn(o);
                }
            }
        }
        if (SPLIT > 1) __syncthreads();                               // s_part is reused by the next iteration
    }
}

template <int WT, int TT, bool SPARSE, bool GATED, int SPLIT, int PAIR>
static int launch_inst(const GemvP & p, size_t smem, cudaStream_t st, bool pdl) {
    // resident CTAs per SM for this instantiation, remembered per (device, shared-memory size) so that replays and
    // stream captures never query the runtime again
    struct Slot { size_t smem; int bps; };
    static Slot cache[16][8] = {};
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) { set_error("gemv: device ordinal %d not supported", dev); return PI_ERR_UNSUPPORTED; }
    auto kern = k_gemv<WT, TT, SPARSE, GATED, SPLIT, PAIR>;
    if (!attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_done[dev] = true;
    }
    int bps = 0;
    for (auto & s : cache[dev]) if (s.bps && s.smem == smem) bps = s.bps;
    if (!bps) {
        PI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&bps, kern, GEMV_THREADS, smem));
        if (bps < 1) { set_error("gemv: activation of %zu bytes does not fit in shared memory", smem); return PI_ERR_INVALID; }
        for (auto & s : cache[dev]) if (!s.bps) { s.smem = smem; s.bps = bps; break; }
    }
    constexpr int items_per_cta = (GEMV_WARPS / SPLIT) * PAIR;
    int grid = sm_count() * bps;
    if (!SPARSE) grid = (int)imin64(grid, (p.nrows + items_per_cta - 1) / items_per_cta);
    if (grid < 1) grid = 1;
    PI_CUDA(launch_k(kern, dim3(grid), dim3(GEMV_THREADS), smem, st, pdl, p));
    return PI_OK;
}

template <int WT, int TT>
static int launch_tt(const GemvP & p, bool sparse, bool gated, size_t smem, cudaStream_t st, bool pdl) {
    if (TT == 1) {
        // batch 1 is latency-bound: stream two items per warp, and split long rows of short matrices over 2 or 4 warps
        // so that enough bytes are in flight (the predictor's fc1 has only `rank` rows of d_model columns)
        if (gated) return launch_inst<WT, 1, true, true, 1, 2>(p, smem, st, pdl);
        if (sparse) return launch_inst<WT, 1, true, false, 1, 2>(p, smem, st, pdl);
        const int unit = WT == PI_TYPE_F16 ? 256 : 32 * 32;          // columns one warp step covers
        const int64_t warps_wanted = (int64_t)sm_count() * 24;
        if (p.nrows * 2 <= warps_wanted && p.ncols % (unit * 4) == 0 && p.ncols >= unit * 16)
            return launch_inst<WT, 1, false, false, 4, 1>(p, smem, st, pdl);
        if (p.nrows <= warps_wanted && p.ncols % (unit * 2) == 0 && p.ncols >= unit * 8)
            return launch_inst<WT, 1, false, false, 2, 1>(p, smem, st, pdl);
        return launch_inst<WT, 1, false, false, 1, 2>(p, smem, st, pdl);
    }
    if (!sparse) return launch_inst<WT, TT, false, false, 1, 1>(p, smem, st, pdl);
    if (gated)   return launch_inst<WT, TT, true, true, 1, 1>(p, smem, st, pdl);
    return launch_inst<WT, TT, true, false, 1, 1>(p, smem, st, pdl);
}

template <int WT>
static int launch_wt(const GemvP & p, int tt, bool sparse, bool gated, size_t smem, cudaStream_t st, bool pdl) {
    switch (tt) {
        case 1: return launch_tt<WT, 1>(p, sparse, gated, smem, st, pdl);
        case 2: return launch_tt<WT, 2>(p, sparse, gated, smem, st, pdl);
        case 4: return launch_tt<WT, 4>(p, sparse, gated, smem, st, pdl);
        default: return launch_tt<WT, 8>(p, sparse, gated, smem, st, pdl);
    }
}

// launch_gemv proper (below) + the activity masks a dense one-token mat-vec was asked for: made by the mat-vec's own
// epilogue where the kernel that runs has one, else by the mask kernel over the result
static int launch_gemv_main(const GemvArgs & a, cudaStream_t st, bool * wrote_masks);

int launch_gemv(const GemvArgs & a, cudaStream_t st) {
    bool wrote = false;
    const int rc = launch_gemv_main(a, st, &wrote);
    if (rc != PI_OK || !a.masks_out || wrote || a.T <= 0 || a.nrows <= 0) return rc;
    if (a.T != 1 || a.list || a.masks || !a.dst) { set_error("gemv: masks_out needs a dense one-token mat-vec with an F32 result"); return PI_ERR_UNSUPPORTED; }
    CompactArgs ca;
    ca.pdl = a.pdl; ca.idx = a.dst; ca.idx_stride = a.dst_stride; ca.T = 1; ca.threshold = a.masks_threshold; ca.n_local = a.nrows;
    ca.masks = a.masks_out;
    return launch_compact(ca, st);
}

static int launch_gemv_main(const GemvArgs & a, cudaStream_t st, bool * wrote_masks) {
    if (a.T <= 0 || a.nrows <= 0) return PI_OK;
    if (a.T == 1 && a.masks) {                                     // one token, rows named by bit masks
        const int rc = launch_gather_rows(a, st);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
        if (!a.list) { set_error("gemv: masks given but the shape is not eligible and there is no list"); return PI_ERR_UNSUPPORTED; }
    }
    if (a.wtype == PI_TYPE_F16 && a.status) {                      // FP16 rows, up to 32 tokens: tensor-core ring kernel
        const int rc = launch_gemv_mma(a, st);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
    }
    if (a.wtype == PI_TYPE_Q4_0 && a.status && a.T > 1) {          // Q4_0 rows, 2+ tokens: integer tensor-core ring kernel
        const int rc = launch_gemv_mma_q4(a, st);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
    }
    if (a.T == 1 && a.status) {
        const int rc = launch_gemv_ring(a, a.status, a.pdl, st, wrote_masks);
        if (rc != PI_ERR_UNSUPPORTED) return rc;
    }
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    const int nb = (int)(a.ncols / QK);
    // tokens are processed in chunks of at most 8 (weights are re-read per chunk; decode batches are <= 32)
    for (int t0 = 0; t0 < a.T; ) {
        const int left = a.T - t0;
        const int tt = left >= 8 ? 8 : (left >= 4 ? 4 : (left >= 2 ? 2 : 1));
        GemvP p;
        p.W = (const uint8_t *)a.W; p.W2 = (const uint8_t *)a.W2;
        p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols);
        p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.nb = nb;
        p.T = tt;
        if (q4) {
            p.x.lo = a.x.lo + (size_t)t0 * nb; p.x.hi = a.x.hi + (size_t)t0 * nb;
            p.x.d = a.x.d + (size_t)t0 * nb;   p.x.s = a.x.s + (size_t)t0 * nb;
        } else {
            p.x.h16 = a.x.h16 + (size_t)t0 * a.ncols;
        }
        p.list = a.list; p.count = a.count; p.bucket = a.bucket;
        p.idx = a.idx ? a.idx + (size_t)t0 * a.idx_stride : nullptr; p.idx_stride = a.idx_stride; p.threshold = a.threshold;
        p.bias = a.bias; p.relu = a.relu;
        p.dst = a.dst ? a.dst + (size_t)t0 * a.dst_stride : nullptr;
        p.dst16 = a.dst16 ? a.dst16 + (size_t)t0 * a.dst_stride : nullptr;
        p.dst_stride = a.dst_stride;
        const size_t smem = q4 ? (size_t)tt * nb * 40 : (size_t)tt * a.ncols * 2;
        const bool sparse = a.list != nullptr;
        const int rc = q4 ? launch_wt<PI_TYPE_Q4_0>(p, tt, sparse, a.W2 != nullptr, smem, st, a.pdl)
                          : launch_wt<PI_TYPE_F16>(p, tt, sparse, a.W2 != nullptr, smem, st, a.pdl);
        if (rc != PI_OK) return rc;
        t0 += tt;
    }
    return PI_OK;
}

}  // namespace pi
