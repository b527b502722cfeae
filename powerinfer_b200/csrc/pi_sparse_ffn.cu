// Batch-1 sparse FFN in one kernel: ggml_mul_mat_idx on up (and gate), the activation, and ggml_axpy on down_t
// (llm_build_ffn_sparse, llama.cpp:4711-4754) over the predicted-active neurons.
//
// One persistent CTA per SM owns a contiguous range of 32-neuron chunks with (nearly) the same number of active rows
// (the split comes from the compaction kernel).  Its rows go through ONE shared-memory ring as a single stream of bulk
// copies (cp.async.bulk + mbarrier, non-tensor, no multicast): first the up / gate rows, then the down_t rows, which do
// not depend on the hidden values and therefore start flying while the dot products are still being computed.
//   pass 1  stage = J row jobs; 32/J warps share one dot product; h[i] = relu(gate.x) * (up.x) | relu(up.x + b)
//   coef    per 32-neuron chunk: the CPU path's axpy coefficient (FP16(h) for FP16 rows; Q8_0 over the chunk for Q4_0)
//   pass 2  1024 threads own fixed columns and add coef * down_t[row] into registers
// Because a chunk never leaves its CTA, the hidden vector never touches global memory and the Q8_0 block statistics are
// local.  Per-CTA partial vectors are summed afterwards in CTA order (fixed order, no atomics).
// Every mbarrier wait is bounded (status bit 3 on expiry, copies drained before exit).
#include "pi_common.cuh"

namespace pi {

static constexpr int QK = 32;
static constexpr int FFN_THREADS = 1024;
static constexpr int FFN_WARPS = 32;
static constexpr int FFN_MAX_ROWS = 512;               // active rows one CTA may own

__device__ __forceinline__ float f_nib(uint32_t bytes, int k) {
    return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650u | (uint32_t)k)) - 8388616.0f;
}
__device__ __forceinline__ int f_block_dot(const uint4 q, const uint4 lo, const uint4 hi, int s8) {
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

struct FfnP {
    const uint8_t * up; const uint8_t * gate; const uint8_t * down;
    int64_t row_bytes; int nrows; int ncols; int nb;
    Act x;
    const uint32_t * masks; const int32_t * parts;
    const float * up_b;
    float * partial; unsigned int * status;
    int J, stages; size_t row_stride;
};

template <int WT, bool GATED, int CPT>
__global__ void __launch_bounds__(FFN_THREADS) k_sparse_ffn(const FfnP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x;
    const int S = p.stages, J = p.J;
    const int NM = GATED ? 2 : 1;

    // shared-memory map
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);                       // [S]
    int *   rows  = reinterpret_cast<int *>(smem + 256);                        // [FFN_MAX_ROWS] neuron ids, ascending
    float * hbuf  = reinterpret_cast<float *>(rows + FFN_MAX_ROWS);             // [FFN_MAX_ROWS] hidden values, then coefficients
    float * dots  = hbuf + FFN_MAX_ROWS;                                        // [2][J][32] per-warp partial dots
    unsigned char * xs = smem + 256 + FFN_MAX_ROWS * 8 + 2 * 32 * 32 * 4;       // staged activation
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * ring = xs + ((x_bytes + 127) & ~(size_t)127);
    const size_t stage_bytes = p.row_stride * J;
    __shared__ int s_nrows;

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    pdl_wait();

    // ---- my chunks -> my rows (ascending neuron id): one warp expands the masks with a running offset
    const int c_lo = p.parts[cta], c_hi = p.parts[cta + 1];
    if (warp == 0) {
        int n = 0;
        for (int c0 = c_lo; c0 < c_hi; c0 += 32) {
            const int c = c0 + lane;
            const uint32_t m = c < c_hi ? __ldcg(p.masks + c) : 0u;
            int incl = __popc(m);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
            int off = n + incl - __popc(m);
            uint32_t mm = m;
            while (mm) {
                const int bit = __ffs(mm) - 1; mm &= mm - 1;
                const int r = c * 32 + bit;
                if (off < FFN_MAX_ROWS) rows[off] = r < p.nrows ? r : 0;
                off++;
            }
            n += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_nrows = min(n, FFN_MAX_ROWS);
    }
    __syncthreads();
    const int n_rows = s_nrows;
    const int jobs1 = n_rows * NM;                      // dot jobs: up_0, gate_0, up_1, gate_1, ... (or up_0, up_1, ...)
    const int jobs = jobs1 + n_rows;                    // then the down rows
    const int n_st1 = (jobs1 + J - 1) / J;              // pass-1 stages (the last may be short)
    const int n_st2 = (n_rows + J - 1) / J;
    const int n_stages = n_st1 + n_st2;
    (void)jobs;
    auto issue = [&](int st) {                          // thread 0 only
        const int s = st % S;
        unsigned char * dstp = ring + (size_t)s * stage_bytes;
        int first, cnt;
        if (st < n_st1) { first = st * J; cnt = min(J, jobs1 - first); }
        else            { first = (st - n_st1) * J; cnt = min(J, n_rows - first); }
        mbar_expect_tx(full + s, (unsigned)(cnt * p.row_bytes));
        for (int k = 0; k < cnt; k++) {
            const uint8_t * src;
            if (st < n_st1) {
                const int job = first + k;
                const int r = rows[GATED ? job >> 1 : job];
                src = ((GATED && (job & 1)) ? p.gate : p.up) + (size_t)r * p.row_bytes;
            } else {
                src = p.down + (size_t)rows[first + k] * p.row_bytes;
            }
            bulk_g2s(dstp + (size_t)k * p.row_stride, src, (unsigned)p.row_bytes, full + s);
        }
    };
    if (tid == 0) for (int st = 0; st < S && st < n_stages; st++) issue(st);

    // ---- stage the activation
    if (WT == PI_TYPE_F16) {
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dstx = reinterpret_cast<uint4 *>(xs);
        for (int i = tid; i < p.ncols / 8; i += FFN_THREADS) dstx[i] = src[i];
    } else {
        uint4 * lo = reinterpret_cast<uint4 *>(xs);
        uint4 * hi = lo + p.nb;
        uint2 * ds = reinterpret_cast<uint2 *>(hi + p.nb);
        for (int i = tid; i < p.nb; i += FFN_THREADS) {
            lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i];
            ds[i] = make_uint2(__float_as_uint(p.x.d[i]), (unsigned)p.x.s[i]);
        }
    }
    __syncthreads();

    // A wait that runs out raises status bit 3 and the thread simply goes on (the stage then holds stale bytes): control flow
    // stays identical in every thread, so no barrier or shuffle below can be left half-populated, and nothing can hang.
    bool dead = false;
    auto wait_stage = [&](int st) {
        const int s = st % S;
        const unsigned parity = (unsigned)(st / S) & 1u;
        int spins = 0;
        while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { dead = true; atomicOr(p.status, 8u); break; } }
    };

    // ---- pass 1: dot products.  W warps share one job; their partial sums meet in shared memory.
    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;
    const int W = FFN_WARPS / J;                        // warps per job
    const int per = (units + W - 1) / W;
    for (int st = 0; st < n_st1; st++) {
        wait_stage(st);
        const unsigned char * base = ring + (size_t)(st % S) * stage_bytes;
        const int first = st * J, cnt = min(J, jobs1 - first);
        const int k = warp / W, part = warp % W;
        float v = 0.f;
        if (k < cnt) {
            const unsigned char * row = base + (size_t)k * p.row_stride;
            const int u_lo = part * per, u_hi = min(units, u_lo + per);
            if (WT == PI_TYPE_F16) {
                const uint4 * w = reinterpret_cast<const uint4 *>(row);
                const uint4 * x = reinterpret_cast<const uint4 *>(xs);
                for (int u = u_lo + lane; u < u_hi; u += 32) {
                    const uint4 wv = w[u], xv = x[u];
                    const float2 w0 = h2f(wv.x), w1 = h2f(wv.y), w2 = h2f(wv.z), w3 = h2f(wv.w);
                    const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
                    v = fmaf(w0.x, x0.x, v); v = fmaf(w0.y, x0.y, v); v = fmaf(w1.x, x1.x, v); v = fmaf(w1.y, x1.y, v);
                    v = fmaf(w2.x, x2.x, v); v = fmaf(w2.y, x2.y, v); v = fmaf(w3.x, x3.x, v); v = fmaf(w3.y, x3.y, v);
                }
            } else {
                const uint4 * q = reinterpret_cast<const uint4 *>(row);
                const __half * sc = reinterpret_cast<const __half *>(row + (size_t)p.nb * 16);
                const uint4 * lo = reinterpret_cast<const uint4 *>(xs);
                const uint4 * hi = lo + p.nb;
                const uint2 * ds = reinterpret_cast<const uint2 *>(hi + p.nb);
                for (int b = u_lo + lane; b < u_hi; b += 32) {
                    const uint2 m = ds[b];
                    v = fmaf((float)f_block_dot(q[b], lo[b], hi[b], (int)m.y), __half2float(sc[b]) * __uint_as_float(m.x), v);
                }
            }
            v = warp_sum(v);
        }
        float * dd = dots + (size_t)(st & 1) * J * 32;
        if (lane == 0) dd[k * 32 + part] = v;
        __syncthreads();                                // stage consumed, partial sums visible
        if (tid == 0 && st + S < n_stages) issue(st + S);
        // finish the rows this stage completed: thread i < rows_done sums its jobs' parts in part order
        const int rows_done = GATED ? cnt / 2 : cnt;    // J is even when GATED, so up/gate pairs never straddle stages
        if (tid < rows_done) {
            float a = 0.f, g = 0.f;
            const int ju = GATED ? 2 * tid : tid;
            for (int q = 0; q < W; q++) a += dd[ju * 32 + q];
            if (GATED) for (int q = 0; q < W; q++) g += dd[(ju + 1) * 32 + q];
            const int i = (GATED ? first / 2 : first) + tid;
            float o = GATED ? fmaxf(g, 0.f) * a : a;
            if (!GATED) { if (p.up_b) o += p.up_b[rows[i]]; o = fmaxf(o, 0.f); }
            hbuf[i] = o;
        }
    }
    __syncthreads();

    // ---- coefficients (ggml.c:14422-14428 FP16; ggml.c:14575-14581 Q4_0: Q8_0 over the 32-neuron chunk)
    {
        if (WT == PI_TYPE_F16) {
            for (int i = tid; i < n_rows; i += FFN_THREADS) hbuf[i] = round_f16(hbuf[i]);
        } else {
            // warp per chunk; lane = neuron of the chunk.  Inactive neurons hold 0 (relu(bias) for the no-gate case with bias).
            int base_i = 0;
            for (int c = c_lo; c < c_hi; c++) {                     // every warp walks all chunks to keep base_i; chunk c is warp (c - c_lo) % 32's
                const uint32_t m = __ldcg(p.masks + c);
                const int cntc = __popc(m);
                if (cntc && ((c - c_lo) & 31) == warp) {
                    const bool act = (m >> lane) & 1u;
                    const int i = base_i + __popc(m & ((1u << lane) - 1u));
                    float hv = 0.f;
                    if (act && i < FFN_MAX_ROWS) hv = hbuf[i];
                    else if (!act && !GATED && p.up_b && c * 32 + lane < p.nrows) hv = fmaxf(p.up_b[c * 32 + lane], 0.f);
                    const float amax = warp_max(fabsf(hv));
                    const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
                    const int q = __float2int_rn(hv * id);
                    __syncwarp();
                    if (act && i < FFN_MAX_ROWS) hbuf[i] = (float)q * round_f16(amax / 127.0f);
                }
                base_i += cntc;
            }
        }
    }
    __syncthreads();

    // ---- pass 2: out += coef * down_t[row]; a thread owns 8 columns (Q4_0: one word of nibbles; FP16: CPT chunks)
    constexpr int NACC = WT == PI_TYPE_F16 ? CPT * 8 : 8;
    float acc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; j++) acc[j] = 0.f;
    const int n_chunks8 = p.ncols / 8, n_words = p.nb * 4;
    for (int st2 = 0; st2 < n_st2; st2++) {
        const int st = n_st1 + st2;
        wait_stage(st);
        const unsigned char * base = ring + (size_t)(st % S) * stage_bytes;
        const int first = st2 * J, cnt = min(J, n_rows - first);
        for (int k = 0; k < cnt; k++) {
            const float c = hbuf[first + k];
            if (c == 0.f) continue;
            const unsigned char * row = base + (size_t)k * p.row_stride;
            if (WT == PI_TYPE_F16) {
#pragma unroll
                for (int q = 0; q < CPT; q++) {
                    const int ch = tid + q * FFN_THREADS;
                    if (ch < n_chunks8) {
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
                const float sc = c * __half2float(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16)[tid >> 2]);
                const uint32_t lo = word & 0x0F0F0F0Fu, hi = (word >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[j]     = fmaf(f_nib(lo, j), sc, acc[j]);
                    acc[4 + j] = fmaf(f_nib(hi, j), sc, acc[4 + j]);
                }
            }
        }
        __syncthreads();
        if (tid == 0 && st + S < n_stages) issue(st + S);
    }
    if (__syncthreads_or(dead) && tid == 0) {             // something timed out: give outstanding copies a bounded chance to land
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }

    float * out = p.partial + (size_t)cta * p.ncols;
    if (WT == PI_TYPE_F16) {
#pragma unroll
        for (int q = 0; q < CPT; q++) {
            const int ch = tid + q * FFN_THREADS;
            if (ch < n_chunks8) {
                *reinterpret_cast<float4 *>(out + ch * 8)     = make_float4(acc[q * 8 + 0], acc[q * 8 + 1], acc[q * 8 + 2], acc[q * 8 + 3]);
                *reinterpret_cast<float4 *>(out + ch * 8 + 4) = make_float4(acc[q * 8 + 4], acc[q * 8 + 5], acc[q * 8 + 6], acc[q * 8 + 7]);
            }
        }
    } else if (tid < n_words) {
        const int b = tid >> 2, i = tid & 3;
        *reinterpret_cast<float4 *>(out + (size_t)b * QK + 4 * i)      = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4 *>(out + (size_t)b * QK + 16 + 4 * i) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

int sparse_ffn_parts() { return sm_count(); }

struct FfnPlan { bool ok; int J, stages, cpt; size_t row_stride, smem; };

static FfnPlan ffn_plan(int wtype, int64_t nrows, int64_t ncols) {
    FfnPlan pl{};
    const size_t row_bytes = pi_row_bytes(wtype, ncols);
    if (row_bytes % 16 != 0) return pl;
    if ((nrows + sparse_ffn_parts() - 1) / sparse_ffn_parts() + 64 > FFN_MAX_ROWS) return pl;     // even a dense mask must fit
    pl.row_stride = (row_bytes + 127) & ~size_t(127);
    if (wtype == PI_TYPE_Q4_0) {
        if (ncols / QK * 4 > FFN_THREADS) return pl;
        pl.cpt = 1;
    } else {
        pl.cpt = (int)((ncols / 8 + FFN_THREADS - 1) / FFN_THREADS);
        if (pl.cpt > 2) return pl;
    }
    // jobs per stage: about 16-32 KB, a power of two in [2, 32] that divides the 32 warps
    int J = 2;
    while (J < 32 && (size_t)(2 * J) * pl.row_stride <= 24 * 1024) J *= 2;
    pl.J = J;
    const size_t x_bytes = wtype == PI_TYPE_F16 ? (size_t)ncols * 2 : (size_t)(ncols / QK) * 40;
    const size_t head = 256 + (size_t)FFN_MAX_ROWS * 8 + 2 * 32 * 32 * 4 + ((x_bytes + 127) & ~size_t(127)) + 128;
    const size_t budget = 200 * 1024;
    const size_t stage_bytes = pl.row_stride * J;
    if (head + 2 * stage_bytes > budget) return pl;
    int S = (int)((budget - head) / stage_bytes);
    pl.stages = S > 16 ? 16 : S;
    pl.smem = head + (size_t)pl.stages * stage_bytes;
    pl.ok = true;
    return pl;
}

template <int WT, bool GATED, int CPT>
static int launch_ffn_inst(const FfnP & p, const FfnPlan & pl, int grid, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_sparse_ffn<WT, GATED, CPT>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(grid), dim3(FFN_THREADS), pl.smem, st, pdl, p));
    return PI_OK;
}

int launch_sparse_ffn(const SparseFfnArgs & a, cudaStream_t st) {
    const FfnPlan pl = ffn_plan(a.wtype, a.nrows, a.ncols);
    if (!pl.ok || !a.status || a.n_parts != sparse_ffn_parts()) return PI_ERR_UNSUPPORTED;
    FfnP p;
    p.up = (const uint8_t *)a.up; p.gate = (const uint8_t *)a.gate; p.down = (const uint8_t *)a.down_t;
    p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols); p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK);
    p.x = a.x; p.masks = a.masks; p.parts = a.parts; p.up_b = a.up_b; p.partial = a.partial; p.status = a.status;
    p.J = pl.J; p.stages = pl.stages; p.row_stride = pl.row_stride;
    const bool q4 = a.wtype == PI_TYPE_Q4_0, gated = a.gate != nullptr;
    const int grid = a.n_parts;
    if (q4) return gated ? launch_ffn_inst<PI_TYPE_Q4_0, true, 1>(p, pl, grid, a.pdl, st) : launch_ffn_inst<PI_TYPE_Q4_0, false, 1>(p, pl, grid, a.pdl, st);
    if (pl.cpt == 1) return gated ? launch_ffn_inst<PI_TYPE_F16, true, 1>(p, pl, grid, a.pdl, st) : launch_ffn_inst<PI_TYPE_F16, false, 1>(p, pl, grid, a.pdl, st);
    return gated ? launch_ffn_inst<PI_TYPE_F16, true, 2>(p, pl, grid, a.pdl, st) : launch_ffn_inst<PI_TYPE_F16, false, 2>(p, pl, grid, a.pdl, st);
}

}  // namespace pi
