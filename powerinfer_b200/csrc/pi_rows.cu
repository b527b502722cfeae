// The two neuron-sparse operators for ONE token, with the weight rows streamed straight into registers.
//
// ggml_mul_mat_idx (gather mat-vec over the active rows of up / gate) and ggml_axpy (scatter-accumulate of the active
// rows of down_t) are HBM-bound gathers of scattered 2-24 KB rows.  Both kernels here take the activity BIT MASKS of the
// predictor (one word per 32 neurons, k_compact's first phase) instead of a compacted list: every CTA scans the few KB of
// masks itself (one L2 round trip, the same a list read would cost), so the serial list-building pass never runs, and
// the rows are dealt to warps by their rank among the active rows, which balances the SMs whatever the mask looks like.
// A lane issues 8-16 independent 128-bit streaming loads per row before it consumes any of them; 16 warps per SM keep
// 70-150 KB in flight per SM without shared-memory staging, barriers in the main loop or waits that could time out.
//
// k_gather_rows: warp per active row (and its gate row), activation staged once per CTA in shared memory, dp4a against
//                Q8_0 planes or FP16 x FP16 products accumulated in FP32 (what the CPU path multiplies), epilogue
//                relu(gate) * up | relu(up + b).
// k_axpy_rows:   CTA = (1024-column slice, row group).  The CTA first makes its own list of rows whose coefficient is not
//                zero (the CPU path skips those too: ggml.c:14422-14428, 14571-14581), so rows that relu zeroed are never
//                fetched; a lane keeps 32 column sums in registers (packed FP32 FMAs), warps are summed in warp order
//                through shared memory, and each row group writes one partial vector: a few dozen partial vectors instead
//                of one per SM, which the next norm (or the exchange) adds in group order.  No atomics: same bits every run.
#include "pi_rows.cuh"

#include <cstdlib>

namespace pi {


// ---------------------------------------------------------------------------------------------- gather mat-vec
struct GatherP {
    const uint8_t * W; const uint8_t * W2;
    int64_t row_bytes; int nrows; int ncols; int nb; int n_chunks;
    Act x;
    const uint32_t * masks; const int32_t * bucket;
    const float * bias; int relu;
    float * dst; unsigned long long * rows_total;
};

// U: 128-bit loads per matrix a lane issues before it consumes any (a row of U * 32 units or fewer is one round trip)
template <int WT, bool GATED, int U>
__global__ void __launch_bounds__(ROWS_THREADS, 1) k_gather_rows(const GatherP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_warp[ROWS_WARPS];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    constexpr int NM = GATED ? 2 : 1;
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * xs = smem;
    uint32_t * s_mask = reinterpret_cast<uint32_t *>(smem + ((x_bytes + 127) & ~(size_t)127));
    int * s_pref = reinterpret_cast<int *>(s_mask + p.n_chunks);

    pdl_launch();
    pdl_wait();
    uint32_t mw[SCAN_WORDS];                                        // the mask words travel while the activation is staged
    scan_masks_load(p.masks, p.n_chunks, p.nrows, mw);
    // ---- stage the activation (FP16 vector, or Q8_0 planes lo | hi | {scale, sum})
    if (WT == PI_TYPE_F16) {
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dstx = reinterpret_cast<uint4 *>(xs);
        for (int i = tid; i < p.ncols / 8; i += ROWS_THREADS) dstx[i] = src[i];
    } else {
        uint4 * lo = reinterpret_cast<uint4 *>(xs);
        uint4 * hi = lo + p.nb;
        uint2 * ds = reinterpret_cast<uint2 *>(hi + p.nb);
        for (int i = tid; i < p.nb; i += ROWS_THREADS) {
            lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i];
            ds[i] = make_uint2(__float_as_uint(p.x.d[i]), (unsigned)p.x.s[i]);
        }
    }
    const int n = scan_masks_finish(mw, p.n_chunks, s_mask, s_pref, s_warp);
    if (p.rows_total && blockIdx.x == 0 && tid == 0 && n) atomicAdd(p.rows_total, (unsigned long long)n);    // statistics
    PI_TL_MARK(0);

    const int TW = gridDim.x * ROWS_WARPS, gw = blockIdx.x * ROWS_WARPS + wid;
    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;       // 16-byte units per row
    for (int base = 0; gw + (long long)base * TW < n; base += 32) {
        // lane l looks up the row of this warp's (base + l)-th rank; ranks grow with l, so the valid lanes are a prefix
        const long long rank = gw + (long long)(base + lane) * TW;
        const int my_row = rank < n ? row_of_rank((int)rank, p.n_chunks, s_mask, s_pref) : -1;
        if (base == 0) PI_TL_MARK(4);
        const int cnt = __popc(__ballot_sync(0xffffffffu, my_row >= 0));
        if (base == 0) PI_TL_MARK(1);
        for (int u0 = 0; u0 < cnt; u0++) {
            const int r = __shfl_sync(0xffffffffu, my_row, u0);
            const uint8_t * row = p.W + (size_t)r * p.row_bytes;
            const uint8_t * row2 = GATED ? p.W2 + (size_t)r * p.row_bytes : nullptr;
            float acc = 0.f, acc2 = 0.f;
            for (int j0 = lane; j0 < units; j0 += 32 * U) {
                uint4 w[U], w2[U];
                __half sc[U], sc2[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u * 32;
                    if (j < units) {
                        w[u] = ldg_stream(reinterpret_cast<const uint4 *>(row) + j);
                        if (GATED) w2[u] = ldg_stream(reinterpret_cast<const uint4 *>(row2) + j);
                        if (WT == PI_TYPE_Q4_0) {
                            sc[u] = __ldg(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16) + j);
                            if (GATED) sc2[u] = __ldg(reinterpret_cast<const __half *>(row2 + (size_t)p.nb * 16) + j);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u * 32;
                    if (j < units) {
                        if (WT == PI_TYPE_F16) {
                            const uint4 xv = reinterpret_cast<const uint4 *>(xs)[j];
                            const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
                            {
                                const float2 w0 = h2f(w[u].x), w1 = h2f(w[u].y), w2_ = h2f(w[u].z), w3 = h2f(w[u].w);
                                acc = fmaf(w0.x, x0.x, acc); acc = fmaf(w0.y, x0.y, acc); acc = fmaf(w1.x, x1.x, acc); acc = fmaf(w1.y, x1.y, acc);
                                acc = fmaf(w2_.x, x2.x, acc); acc = fmaf(w2_.y, x2.y, acc); acc = fmaf(w3.x, x3.x, acc); acc = fmaf(w3.y, x3.y, acc);
                            }
                            if (GATED) {
                                const float2 w0 = h2f(w2[u].x), w1 = h2f(w2[u].y), w2_ = h2f(w2[u].z), w3 = h2f(w2[u].w);
                                acc2 = fmaf(w0.x, x0.x, acc2); acc2 = fmaf(w0.y, x0.y, acc2); acc2 = fmaf(w1.x, x1.x, acc2); acc2 = fmaf(w1.y, x1.y, acc2);
                                acc2 = fmaf(w2_.x, x2.x, acc2); acc2 = fmaf(w2_.y, x2.y, acc2); acc2 = fmaf(w3.x, x3.x, acc2); acc2 = fmaf(w3.y, x3.y, acc2);
                            }
                        } else {
                            const uint4 * lo = reinterpret_cast<const uint4 *>(xs);
                            const uint4 * hi = lo + p.nb;
                            const uint2 m = reinterpret_cast<const uint2 *>(hi + p.nb)[j];
                            const uint4 l = lo[j], h = hi[j];
                            const float d8 = __uint_as_float(m.x);
                            acc = fmaf((float)q4_block_dot(w[u], l, h, (int)m.y), __half2float(sc[u]) * d8, acc);
                            if (GATED) acc2 = fmaf((float)q4_block_dot(w2[u], l, h, (int)m.y), __half2float(sc2[u]) * d8, acc2);
                        }
                    }
                }
            }
            acc = warp_sum(acc);
            if (GATED) acc2 = warp_sum(acc2);
            if (base == 0 && u0 == 0) PI_TL_MARK(2);
            if (lane == 0) {
                const int64_t g = p.bucket ? p.bucket[r] : r;
                float o = acc;                                       // one token: a row named by the mask is an active row
                if (GATED) o = fmaxf(acc2, 0.f) * acc;
                if (p.bias) o += p.bias[g];
                if (p.relu) o = fmaxf(o, 0.f);
                p.dst[g] = o;
            }
        }
    }
}

static size_t gather_smem(int wtype, int64_t ncols, int n_chunks) {
    const size_t x_bytes = wtype == PI_TYPE_F16 ? (size_t)ncols * 2 : (size_t)(ncols / QK) * 40;
    return ((x_bytes + 127) & ~size_t(127)) + (size_t)(2 * n_chunks + 1) * 4 + 128;
}

template <int WT, bool GATED, int U>
static int launch_gather_u(const GatherP & p, size_t smem, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_gather_rows<WT, GATED, U>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(sm_count()), dim3(ROWS_THREADS), smem, st, pdl, p));
    return PI_OK;
}

template <int WT, bool GATED>
static int launch_gather_inst(const GatherP & p, size_t smem, bool pdl, cudaStream_t st) {
    if (WT == PI_TYPE_F16) return launch_gather_u<WT, GATED, 8>(p, smem, pdl, st);
    // Q4_0: 9 loads per lane where that saves a round trip per row (rows of 257..288 blocks: d_model 8192 + its scales)
    const int units = p.nb;
    if ((units + 287) / 288 < (units + 255) / 256) return launch_gather_u<WT, GATED, 9>(p, smem, pdl, st);
    return launch_gather_u<WT, GATED, 8>(p, smem, pdl, st);
}

static void axpy_rows_shape(int64_t nrows, int64_t ncols, int * n_slices, int * n_rg, int * max_rows);
static size_t axpy_rows_smem(int n_chunks, int max_rows);

// shapes both kernels take: the masks fit one CTA's scan, rows are 16-byte multiples, shared memory suffices
bool rows_eligible(int wtype, int64_t nrows, int64_t ncols) {
    static int enabled = -1;                                        // PI_ROWS=0: the list-driven kernels instead (diagnostic)
    if (enabled < 0) { const char * v = getenv("PI_ROWS"); enabled = !(v && v[0] == '0'); }
    if (!enabled) return false;
    const int64_t n_chunks = (nrows + 31) / 32;
    if (n_chunks > ROWS_MAX_CHUNKS || nrows <= 0 || ncols <= 0) return false;
    if (pi_row_bytes(wtype, ncols) % 16 != 0) return false;
    if (gather_smem(wtype, ncols, (int)n_chunks) > 160 * 1024) return false;
    int ns, rg, mr;
    axpy_rows_shape(nrows, ncols, &ns, &rg, &mr);
    return mr <= AXPY_MAX_CTA_ROWS && axpy_rows_smem((int)n_chunks, mr) <= 160 * 1024;
}

int launch_gather_rows(const GemvArgs & a, cudaStream_t st) {
    if (a.T != 1 || !a.masks || !a.dst || a.dst16 || !rows_eligible(a.wtype, a.nrows, a.ncols))
        return PI_ERR_UNSUPPORTED;
    GatherP p;
    p.W = (const uint8_t *)a.W; p.W2 = (const uint8_t *)a.W2; p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols);
    p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK); p.n_chunks = (int)((a.nrows + 31) / 32);
    p.x = a.x; p.masks = a.masks; p.bucket = a.bucket; p.bias = a.bias; p.relu = a.relu; p.dst = a.dst;
    p.rows_total = a.rows_total;
    const size_t smem = gather_smem(a.wtype, a.ncols, p.n_chunks);
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    if (a.W2) return q4 ? launch_gather_inst<PI_TYPE_Q4_0, true>(p, smem, a.pdl, st) : launch_gather_inst<PI_TYPE_F16, true>(p, smem, a.pdl, st);
    return q4 ? launch_gather_inst<PI_TYPE_Q4_0, false>(p, smem, a.pdl, st) : launch_gather_inst<PI_TYPE_F16, false>(p, smem, a.pdl, st);
}

// ---------------------------------------------------------------------------------------------- axpy
struct AxpyRowsP {
    const uint8_t * Wt; int64_t row_bytes; int nrows; int ncols; int nb; int n_chunks;
    const float * h; const uint32_t * masks; const int32_t * bucket; int h_uncleared;
    float * partial; int n_slices; int n_rg; int max_rows;
};


template <int WT>
__global__ void __launch_bounds__(ROWS_THREADS, 1) k_axpy_rows(const AxpyRowsP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_warp[ROWS_WARPS];
    __shared__ int s_cnt;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int slice = blockIdx.x % p.n_slices, rg = blockIdx.x / p.n_slices;
    // shared-memory map: masks | prefix | rows of this CTA | their coefficients | (later, over all of it) the warps' sums
    uint32_t * s_mask = reinterpret_cast<uint32_t *>(smem);
    int * s_pref = reinterpret_cast<int *>(s_mask + p.n_chunks);
    int * s_row = s_pref + p.n_chunks + 1;
    float * s_coef = reinterpret_cast<float *>(s_row + p.max_rows);

    pdl_launch();
    pdl_wait();
    const int n = scan_masks(p.masks, p.n_chunks, p.nrows, s_mask, s_pref, s_warp);
    PI_TL_MARK(0);

    // ---- the rows of this row group (ranks rg, rg + n_rg, ...) whose coefficient is not zero, in rank order.
    // Coefficient = what the CPU path multiplies the row by: FP16(h) for FP16 rows; for Q4_0 the int8 quant of h within its
    // block of 32 neurons times that block's FP16 scale (ggml.c:14575-14581, quantize_row_q8_0).
    const int n_mine = rg < n ? min((n - rg + p.n_rg - 1) / p.n_rg, p.max_rows) : 0;
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (int t0 = 0; t0 < n_mine; t0 += ROWS_THREADS) {
        const int t = t0 + tid;
        int r = -1; float c = 0.f;
        if (t < n_mine) {
            r = row_of_rank(rg + t * p.n_rg, p.n_chunks, s_mask, s_pref);
            if (t0 == 0) PI_TL_MARK(4);
            const int64_t g = p.bucket ? p.bucket[r] : r;
            if (WT == PI_TYPE_F16) {
                c = round_f16(__ldcg(p.h + g));
            } else {
                const float4 * hb = reinterpret_cast<const float4 *>(p.h + (g & ~(int64_t)31));
                float4 v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) v[k] = __ldcg(hb + k);
                if (p.h_uncleared) {                                // nobody cleared h where a row is inactive: those entries count as 0
                    const uint32_t mk = s_mask[r >> 5];
#pragma unroll
                    for (int k = 0; k < 8; k++) {
                        if (!(mk >> (4 * k) & 1u))     v[k].x = 0.f;
                        if (!(mk >> (4 * k + 1) & 1u)) v[k].y = 0.f;
                        if (!(mk >> (4 * k + 2) & 1u)) v[k].z = 0.f;
                        if (!(mk >> (4 * k + 3) & 1u)) v[k].w = 0.f;
                    }
                }
                float amax = 0.f;
#pragma unroll
                for (int k = 0; k < 8; k++) amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w))));
                const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
                const float mine = __ldcg(p.h + g);
                c = (float)__float2int_rn(mine * id) * round_f16(amax / 127.0f);
            }
        }
        // keep the order: ballot inside the warp, warp offsets through shared memory
        if (t0 == 0) PI_TL_MARK(5);
        const bool keep = r >= 0 && c != 0.f;
        const unsigned bal = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) s_warp[wid] = __popc(bal);
        __syncthreads();
        int off = s_cnt;
        for (int w = 0; w < wid; w++) off += s_warp[w];
        if (keep) { const int o = off + __popc(bal & ((1u << lane) - 1u)); s_row[o] = r; s_coef[o] = c; }
        __syncthreads();
        if (tid == 0) { int tot = 0; for (int w = 0; w < ROWS_WARPS; w++) tot += s_warp[w]; s_cnt += tot; }
        __syncthreads();
    }
    const int m = s_cnt;
    PI_TL_MARK(1);

    // ---- main loop: warp w takes entries w, w + 16, ...; a lane owns 32 columns of the slice:
    //      Q4_0: block `slice * 32 + lane` (sum index = column inside the block);
    //      FP16: 8 columns at 8 * lane of each of the slice's four 256-column quarters (sum index = 8 * quarter + e).
    constexpr int U = WT == PI_TYPE_F16 ? 4 : 8;                    // rows in flight per warp
    unsigned long long acc[16];
#pragma unroll
    for (int j = 0; j < 16; j++) acc[j] = 0ull;
    float corr = 0.f;
    const int unit0 = WT == PI_TYPE_F16 ? slice * (SLICE / 8) + lane : slice * 32 + lane;
    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;
    for (int i0 = wid; i0 < m; i0 += ROWS_WARPS * U) {
        if (WT == PI_TYPE_Q4_0) {
            uint4 q[U]; __half d4[U]; float c[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = i0 + u * ROWS_WARPS;
                c[u] = 0.f; q[u] = make_uint4(0u, 0u, 0u, 0u); d4[u] = __ushort_as_half((unsigned short)0);
                if (i < m && unit0 < units) {
                    const uint8_t * row = p.Wt + (size_t)s_row[i] * p.row_bytes;
                    c[u] = s_coef[i];
                    q[u] = ldg_stream(reinterpret_cast<const uint4 *>(row) + unit0);
                    d4[u] = __ldg(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16) + unit0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                // nibble q -> the float 16 + q with one byte permute (q lands in mantissa bits 19..22 under the exponent of
                // 16); (q - 8) * sc = (16 + q) * sc - 24 * sc, and the second term is summed once per row instead of once
                // per weight (costs under 2 bits of the FP32 accumulator)
                const float sc = c[u] * __half2float(d4[u]);
                corr += sc;
                const unsigned long long sc2 = pack2(sc, sc);
                const uint32_t wds[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
                for (int wi = 0; wi < 4; wi++) {
                    const uint32_t lo = ((wds[wi] << 3) & 0x78787878u) | 0x80808080u;
                    const uint32_t hi = ((wds[wi] >> 1) & 0x78787878u) | 0x80808080u;
                    const unsigned long long l01 = (unsigned long long)__byte_perm(lo, 0x41000000u, 0x7044u) | ((unsigned long long)__byte_perm(lo, 0x41000000u, 0x7144u) << 32);
                    const unsigned long long l23 = (unsigned long long)__byte_perm(lo, 0x41000000u, 0x7244u) | ((unsigned long long)__byte_perm(lo, 0x41000000u, 0x7344u) << 32);
                    const unsigned long long h01 = (unsigned long long)__byte_perm(hi, 0x41000000u, 0x7044u) | ((unsigned long long)__byte_perm(hi, 0x41000000u, 0x7144u) << 32);
                    const unsigned long long h23 = (unsigned long long)__byte_perm(hi, 0x41000000u, 0x7244u) | ((unsigned long long)__byte_perm(hi, 0x41000000u, 0x7344u) << 32);
                    ffma2(acc[wi * 2], l01, sc2); ffma2(acc[wi * 2 + 1], l23, sc2);
                    ffma2(acc[8 + wi * 2], h01, sc2); ffma2(acc[8 + wi * 2 + 1], h23, sc2);
                }
            }
        } else {
            uint4 w[U][4]; float c[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int i = i0 + u * ROWS_WARPS;
                c[u] = 0.f;
#pragma unroll
                for (int k = 0; k < 4; k++) w[u][k] = make_uint4(0u, 0u, 0u, 0u);
                if (i < m) {
                    const uint4 * row = reinterpret_cast<const uint4 *>(p.Wt + (size_t)s_row[i] * p.row_bytes);
                    c[u] = s_coef[i];
#pragma unroll
                    for (int k = 0; k < 4; k++) if (unit0 + k * 32 < units) w[u][k] = ldg_stream(row + unit0 + k * 32);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const unsigned long long c2 = pack2(c[u], c[u]);
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 f0 = h2f(w[u][k].x), f1 = h2f(w[u][k].y), f2 = h2f(w[u][k].z), f3 = h2f(w[u][k].w);
                    ffma2(acc[k * 4 + 0], pack2(f0.x, f0.y), c2); ffma2(acc[k * 4 + 1], pack2(f1.x, f1.y), c2);
                    ffma2(acc[k * 4 + 2], pack2(f2.x, f2.y), c2); ffma2(acc[k * 4 + 3], pack2(f3.x, f3.y), c2);
                }
            }
        }
    }

    // ---- warps are added in warp order through shared memory (sum index a of lane l at a * 33 + l: no bank conflicts),
    //      then the slice of this row group's partial vector is written
    __syncthreads();                                                 // everyone is done with s_row / s_coef
    PI_TL_MARK(2);
    float * s_red = reinterpret_cast<float *>(smem);
    float * mine = s_red + (size_t)wid * (32 * 33);
#pragma unroll
    for (int j = 0; j < 16; j++) {
        float a0 = lo_f(acc[j]), a1 = hi_f(acc[j]);
        if (WT == PI_TYPE_Q4_0) { a0 = fmaf(-24.0f, corr, a0); a1 = fmaf(-24.0f, corr, a1); }
        mine[(2 * j) * 33 + lane] = a0;
        mine[(2 * j + 1) * 33 + lane] = a1;
    }
    __syncthreads();
    PI_TL_MARK(3);
    float * out = p.partial + (size_t)rg * p.ncols + (size_t)slice * SLICE;
    for (int cidx = tid; cidx < SLICE; cidx += ROWS_THREADS) {
        if ((size_t)slice * SLICE + cidx >= (size_t)p.ncols) break;
        int a, l;
        if (WT == PI_TYPE_Q4_0) { l = cidx >> 5; a = cidx & 31; }
        else                    { const int q = cidx >> 8; l = (cidx & 255) >> 3; a = q * 8 + (cidx & 7); }
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ROWS_WARPS; w++) v += s_red[(size_t)w * (32 * 33) + a * 33 + l];
        out[cidx] = v;
    }
}

static void axpy_rows_shape(int64_t nrows, int64_t ncols, int * n_slices, int * n_rg, int * max_rows) {
    const int ns = (int)((ncols + SLICE - 1) / SLICE);
    int rg = sm_count() / ns;
    rg = rg < 1 ? 1 : (rg > 40 ? 40 : rg);
    *n_slices = ns; *n_rg = rg; *max_rows = (int)((nrows + rg - 1) / rg);
}

static size_t axpy_rows_smem(int n_chunks, int max_rows) {
    const size_t lists = (size_t)(2 * n_chunks + 1) * 4 + (size_t)max_rows * 8;
    const size_t red = (size_t)ROWS_WARPS * 32 * 33 * 4;
    return (lists > red ? lists : red) + 128;
}

int axpy_rows_groups(int64_t nrows, int64_t ncols) {
    int ns, rg, mr;
    axpy_rows_shape(nrows, ncols, &ns, &rg, &mr);
    return rg;
}

template <int WT>
static int launch_axpy_rows_inst(const AxpyRowsP & p, size_t smem, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_axpy_rows<WT>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(p.n_slices * p.n_rg), dim3(ROWS_THREADS), smem, st, pdl, p));
    return PI_OK;
}

int launch_axpy_rows(const AxpyArgs & a, cudaStream_t st, int * groups_used) {
    if (a.T != 1 || !a.masks || !rows_eligible(a.wtype, a.nrows, a.ncols)) return PI_ERR_UNSUPPORTED;
    if (a.h_uncleared && a.bucket) return PI_ERR_UNSUPPORTED;          // the masks are by local row, h by global id
    AxpyRowsP p;
    axpy_rows_shape(a.nrows, a.ncols, &p.n_slices, &p.n_rg, &p.max_rows);
    if (p.max_rows > AXPY_MAX_CTA_ROWS || p.n_rg > a.n_groups) return PI_ERR_UNSUPPORTED;
    p.Wt = (const uint8_t *)a.Wt; p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols); p.nrows = (int)a.nrows;
    p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK); p.n_chunks = (int)((a.nrows + 31) / 32);
    p.h = a.h; p.masks = a.masks; p.bucket = a.bucket; p.h_uncleared = a.h_uncleared ? 1 : 0; p.partial = a.partial;
    const size_t smem = axpy_rows_smem(p.n_chunks, p.max_rows);
    if (smem > 160 * 1024) return PI_ERR_UNSUPPORTED;
    if (groups_used) *groups_used = p.n_rg;
    return a.wtype == PI_TYPE_Q4_0 ? launch_axpy_rows_inst<PI_TYPE_Q4_0>(p, smem, a.pdl, st)
                                   : launch_axpy_rows_inst<PI_TYPE_F16>(p, smem, a.pdl, st);
}

}  // namespace pi
