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
static constexpr int UNROLL = 4;

struct GemvP {
    const uint8_t * W; const uint8_t * W2;
    int64_t row_bytes; int nrows; int ncols; int nb;
    Act x; int T;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; int64_t idx_stride; float threshold;
    const float * bias; int relu;
    float * dst; __half * dst16; int64_t dst_stride;
};

// dot of one FP16 row with TT staged FP16 activation vectors
template <int TT>
__device__ __forceinline__ void row_dot_f16(const uint8_t * __restrict__ row, int ncols, const __half * __restrict__ xs,
                                            int lane, float (&acc)[TT]) {
    for (int c0 = lane * 8; c0 < ncols; c0 += 256 * UNROLL) {
        uint4 w[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int c = c0 + u * 256;
            if (c < ncols) w[u] = ldg_stream(row + (size_t)c * 2);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int c = c0 + u * 256;
            if (c < ncols) {
                const float2 w0 = h2f(w[u].x), w1 = h2f(w[u].y), w2 = h2f(w[u].z), w3 = h2f(w[u].w);
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    const uint4 xv = *reinterpret_cast<const uint4 *>(xs + (size_t)t * ncols + c);
                    const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
                    float a = acc[t];
                    a = fmaf(w0.x, x0.x, a); a = fmaf(w0.y, x0.y, a);
                    a = fmaf(w1.x, x1.x, a); a = fmaf(w1.y, x1.y, a);
                    a = fmaf(w2.x, x2.x, a); a = fmaf(w2.y, x2.y, a);
                    a = fmaf(w3.x, x3.x, a); a = fmaf(w3.y, x3.y, a);
                    acc[t] = a;
                }
            }
        }
    }
}

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

struct SmemQ8 {            // staged Q8_0 planes of TT tokens
    const uint4 * lo; const uint4 * hi; const float * d; const int * s;
};

template <int TT>
__device__ __forceinline__ void row_dot_q4(const uint8_t * __restrict__ row, int nb, const SmemQ8 xs, int lane,
                                           float (&acc)[TT]) {
    const uint4 * qrow = reinterpret_cast<const uint4 *>(row);
    const __half * srow = reinterpret_cast<const __half *>(row + (size_t)nb * 16);
    for (int b0 = lane; b0 < nb; b0 += 32 * UNROLL) {
        uint4 q[UNROLL];
        __half sc[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int b = b0 + u * 32;
            if (b < nb) { q[u] = ldg_stream(qrow + b); sc[u] = __ldg(srow + b); }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int b = b0 + u * 32;
            if (b < nb) {
                const float d4 = __half2float(sc[u]);
#pragma unroll
                for (int t = 0; t < TT; t++) {
                    const int i = t * nb + b;
                    const int sumi = block_dot_q4_q8(q[u], xs.lo[i], xs.hi[i], xs.s[i]);
                    acc[t] = fmaf((float)sumi, d4 * xs.d[i], acc[t]);
                }
            }
        }
    }
}

template <int WT, int TT, bool SPARSE, bool GATED>
__global__ void __launch_bounds__(GEMV_THREADS) k_gemv(const GemvP p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31;

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

    const int warps_total = gridDim.x * (GEMV_THREADS / 32);
    const int gw = blockIdx.x * (GEMV_THREADS / 32) + (tid >> 5);
    const int n_items = SPARSE ? min(*p.count, p.nrows) : p.nrows;

    for (int it = gw; it < n_items; it += warps_total) {
        const int r = SPARSE ? p.list[it] : it;
        if (SPARSE && (unsigned)r >= (unsigned)p.nrows) continue;       // a damaged list must not turn into a wild read
        float acc[TT], acc2[TT];
#pragma unroll
        for (int t = 0; t < TT; t++) { acc[t] = 0.f; acc2[t] = 0.f; }
        const uint8_t * row = p.W + (size_t)r * p.row_bytes;
        if (WT == PI_TYPE_F16) {
            row_dot_f16<TT>(row, p.ncols, xh, lane, acc);
            if (GATED) row_dot_f16<TT>(p.W2 + (size_t)r * p.row_bytes, p.ncols, xh, lane, acc2);
        } else {
            row_dot_q4<TT>(row, p.nb, xq, lane, acc);
            if (GATED) row_dot_q4<TT>(p.W2 + (size_t)r * p.row_bytes, p.nb, xq, lane, acc2);
        }
#pragma unroll
        for (int t = 0; t < TT; t++) { acc[t] = warp_sum(acc[t]); if (GATED) acc2[t] = warp_sum(acc2[t]); }

        const int64_t g = SPARSE && p.bucket ? p.bucket[r] : r;
        if (lane < TT) {
            float v = 0.f, v2 = 0.f;
#pragma unroll
            for (int t = 0; t < TT; t++) if (lane == t) { v = acc[t]; v2 = acc2[t]; }
            const int t = lane;
            bool active = true;
            if (SPARSE) active = p.idx[(size_t)t * p.idx_stride + g] >= p.threshold;
            float o = active ? v : 0.f;
            if (GATED) o = active ? fmaxf(v2, 0.f) * v : 0.f;
            if (p.bias) o += p.bias[g];
            if (p.relu) o = fmaxf(o, 0.f);
            if (p.dst)   p.dst[(size_t)t * p.dst_stride + g] = o;
            if (p.dst16) p.dst16[(size_t)t * p.dst_stride + g] = __float2half_rn(o);
        }
    }
}

template <int WT, int TT, bool SPARSE, bool GATED>
static int launch_inst(const GemvP & p, size_t smem, cudaStream_t st) {
    // resident CTAs per SM for this instantiation, remembered per (device, shared-memory size) so that replays and
    // stream captures never query the runtime again
    struct Slot { size_t smem; int bps; };
    static Slot cache[16][8] = {};
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 16) { set_error("gemv: device ordinal %d not supported", dev); return PI_ERR_UNSUPPORTED; }
    auto kern = k_gemv<WT, TT, SPARSE, GATED>;
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
    const int warps_per_block = GEMV_THREADS / 32;
    int grid = sm_count() * bps;
    if (!SPARSE) grid = (int)imin64(grid, (p.nrows + warps_per_block - 1) / warps_per_block);
    if (grid < 1) grid = 1;
    kern<<<grid, GEMV_THREADS, smem, st>>>(p);
    PI_LAUNCH_CHECK("k_gemv");
    return PI_OK;
}

template <int WT, int TT>
static int launch_tt(const GemvP & p, bool sparse, bool gated, size_t smem, cudaStream_t st) {
    if (!sparse) return launch_inst<WT, TT, false, false>(p, smem, st);
    if (gated)   return launch_inst<WT, TT, true, true>(p, smem, st);
    return launch_inst<WT, TT, true, false>(p, smem, st);
}

template <int WT>
static int launch_wt(const GemvP & p, int tt, bool sparse, bool gated, size_t smem, cudaStream_t st) {
    switch (tt) {
        case 1: return launch_tt<WT, 1>(p, sparse, gated, smem, st);
        case 2: return launch_tt<WT, 2>(p, sparse, gated, smem, st);
        case 4: return launch_tt<WT, 4>(p, sparse, gated, smem, st);
        default: return launch_tt<WT, 8>(p, sparse, gated, smem, st);
    }
}

int launch_gemv(const GemvArgs & a, cudaStream_t st) {
    if (a.T <= 0 || a.nrows <= 0) return PI_OK;
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
        const int rc = q4 ? launch_wt<PI_TYPE_Q4_0>(p, tt, sparse, a.W2 != nullptr, smem, st)
                          : launch_wt<PI_TYPE_F16>(p, tt, sparse, a.W2 != nullptr, smem, st);
        if (rc != PI_OK) return rc;
        t0 += tt;
    }
    return PI_OK;
}

}  // namespace pi
