// The whole neuron-sparse FFN of ONE token in one launch: ggml_mul_mat_idx over the active rows of up / gate, the
// activation, and ggml_axpy over the same rows of down_t (llama.cpp:4697-4760 builds them as three graph nodes).
//
// Two separate kernels pay the launch boundary, the mask scan and the trip of the hidden vector through L2 twice, and
// their last wave runs with most warps idle.  Here a thread-block CLUSTER owns a contiguous range of whole 32-neuron
// blocks holding 1 / n_clusters of the active rows (every CTA finds the range itself from the scanned masks):
//   gather  the cluster's rows are split evenly over its CTAs, and a CTA's rows over its 16 warps BY 16-BYTE UNITS, so a
//           warp streams the same number of bytes whatever the rows look like (a row may be shared by two warps; the
//           pieces meet in shared memory and are added in warp order);
//   hand-over  the activations go to every CTA of the cluster through distributed shared memory (one cluster barrier;
//           nothing goes through L2 and no other cluster is waited for);
//   axpy    CTA j of the cluster takes the 1024-column slices j, j + cluster size, ... of down_t over the cluster's rows
//           whose coefficient is not zero (the CPU path skips those too: ggml.c:14422-14428, 14571-14581); the Q4_0
//           coefficient needs the largest |h| of a row's 32-neuron block, which is why ranges are whole blocks.
// Each cluster writes one partial vector; the next norm adds them in cluster order.  No atomics, no waits that could
// time out: same bits every run.
#include "pi_rows.cuh"

#include <cstdio>
#include <cstdlib>

namespace pi {

struct FfnRowsP {
    const uint8_t * Wup; const uint8_t * Wgate; const uint8_t * Wdown;
    int64_t row_bytes; int nrows; int ncols; int nb; int n_chunks;
    Act x; const uint32_t * masks;
    const float * bias; int relu;
    float * h_out; float * partial; unsigned long long * rows_total;
    int n_clusters; int cap; int cap_cta;
};

__device__ __forceinline__ unsigned cl_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cl_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cl_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cl_wait()   { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// store into the same shared-memory variable of CTA `rank` of this cluster
__device__ __forceinline__ void cl_store_u32(const void * local, unsigned rank, uint32_t v) {
    unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(ra), "r"(v) : "memory");
}

static __host__ __device__ __forceinline__ size_t up128(size_t v) { return (v + 127) & ~(size_t)127; }

// NS: 1024-column slices of down_t a CTA works on at a time (2 when a CTA owns more than one: their loads travel together)
template <int WT, bool GATED, int U, int NS>
__global__ void __launch_bounds__(ROWS_THREADS, 1) k_ffn_rows(const FfnRowsP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_warp[ROWS_WARPS];
    __shared__ int s_cnt;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int CS = (int)cl_size(), cj = (int)cl_rank();
    const int cluster = blockIdx.x / CS;
    constexpr int NM = GATED ? 2 : 1;
    // ---- shared-memory map.  Lists that live for the whole kernel, then a region used first for the staged activation and
    //      the pieces of the gather, later for the warps' column sums.
    uint32_t * s_mask = reinterpret_cast<uint32_t *>(smem);
    int *   s_pref  = reinterpret_cast<int *>(s_mask + p.n_chunks);
    float * s_h     = reinterpret_cast<float *>(s_pref + p.n_chunks + 1);   // [cap] activations of the cluster's rows, by rank
    int *   s_rowc  = reinterpret_cast<int *>(s_h + p.cap);                 // [cap] their row numbers
    int *   s_row2  = s_rowc + p.cap;                                       // [cap] rows with a coefficient != 0 ...
    float * s_coef  = reinterpret_cast<float *>(s_row2 + p.cap);            // [cap] ... and the coefficients
    int *   s_myrow = reinterpret_cast<int *>(s_coef + p.cap);              // [cap_cta] rows this CTA gathers
    unsigned char * region = smem + up128((size_t)(2 * p.n_chunks + 1) * 4 + (size_t)p.cap * 16 + (size_t)p.cap_cta * 4);
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * xs = region;
    float * s_part = reinterpret_cast<float *>(region + up128(x_bytes));    // [cap_cta][ROWS_WARPS][NM]
    float * s_red  = reinterpret_cast<float *>(region);                     // [NS][ROWS_WARPS][32 * 33]

    pdl_launch();
    pdl_wait();
    uint32_t mw[SCAN_WORDS];                                        // the mask words travel while the activation is staged
    scan_masks_load(p.masks, p.n_chunks, p.nrows, mw);
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
    cl_arrive();                                                     // (waited for before the first store into a peer's memory)
    PI_TL_MARK(0);

    // ---- this cluster's range of mask words [kb, ke): from the first word at which the running count reaches the cluster's
    //      share c * n / n_clusters.  Every thread looks at the words it scanned; exactly one word (or none: then the end of
    //      the masks) is the first to reach a target.
    __shared__ int s_kb, s_ke;
    if (tid == 0) { s_kb = p.n_chunks; s_ke = p.n_chunks; }
    __syncthreads();
    {
        const unsigned tb = (unsigned)cluster * (unsigned)n / (unsigned)p.n_clusters;               // n * n_clusters < 2^31
        const unsigned te = (unsigned)(cluster + 1) * (unsigned)n / (unsigned)p.n_clusters;
        const bool last = cluster + 1 >= p.n_clusters;
        const int per = (p.n_chunks + ROWS_THREADS - 1) / ROWS_THREADS;
        const int c0 = min(tid * per, p.n_chunks), c1 = min(c0 + per, p.n_chunks);
        for (int k = c0; k < c1; k++) {
            const unsigned here = (unsigned)s_pref[k];
            const bool first_word = k == 0;
            const unsigned before = first_word ? 0u : (unsigned)s_pref[k - 1];
            if (here >= tb && (first_word || before < tb)) s_kb = k;
            if (!last && here >= te && (first_word || before < te)) s_ke = k;
        }
    }
    __syncthreads();
    const int kb = s_kb, ke = s_ke;
    const int r0 = s_pref[kb];
    const int m = min(s_pref[ke] - r0, p.cap);                       // < n / n_clusters + 34 <= cap by the launcher's choice of cap

    // ================================================================= gather: rows [i0, i1) of the cluster, by units
    const int i0 = (int)((unsigned)cj * (unsigned)m / (unsigned)CS), i1 = (int)((unsigned)(cj + 1) * (unsigned)m / (unsigned)CS);
    const int mj = min(i1 - i0, p.cap_cta);
    {
        // the rows of this CTA: every thread expands the bits of the words it scanned whose ranks fall into [r0 + i0, r0 + i0 + mj)
        const int lo_rank = r0 + i0, hi_rank = lo_rank + mj;
        const int per = (p.n_chunks + ROWS_THREADS - 1) / ROWS_THREADS;
        const int c0 = max(min(tid * per, p.n_chunks), kb), c1 = min(min(tid * per + per, p.n_chunks), ke);
        for (int k = c0; k < c1; k++) {
            int rank = s_pref[k];
            uint32_t mk = s_mask[k];
            if (rank >= hi_rank || rank + __popc(mk) <= lo_rank) continue;
            while (mk) {
                const int bit = __ffs(mk) - 1;
                mk &= mk - 1;
                if (rank >= lo_rank && rank < hi_rank) s_myrow[rank - lo_rank] = k * 32 + bit;
                rank++;
            }
        }
    }
    for (int t = tid; t < mj * ROWS_WARPS * NM; t += ROWS_THREADS) s_part[t] = 0.f;
    __syncthreads();
    PI_TL_MARK(1);
    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;       // 16-byte units per row
    {
        // The CTA's rows laid end to end are mj * units 16-byte units; warp w streams the w-th sixteenth of them, piece by
        // piece (a piece = the part of one row inside the warp's range), so every warp moves the same number of bytes.
        const unsigned tot = (unsigned)mj * (unsigned)units;                              // < 2^24
        unsigned cur = (unsigned)wid * tot / ROWS_WARPS;
        const unsigned end = (unsigned)(wid + 1) * tot / ROWS_WARPS;
        while (cur < end) {
            const int rl = (int)(cur / (unsigned)units), ub = (int)(cur % (unsigned)units);
            const int ue = (int)min((unsigned)units, (unsigned)ub + (end - cur));
            const int r = s_myrow[rl];
            const uint8_t * row = p.Wup + (size_t)r * p.row_bytes;
            const uint8_t * row2 = GATED ? p.Wgate + (size_t)r * p.row_bytes : nullptr;
            float acc = 0.f, acc2 = 0.f;
            for (int j0 = ub + lane; j0 < ue; j0 += 32 * U) {
                uint4 w[U], w2[U];
                __half sc[U], sc2[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int j = j0 + u * 32;
                    if (j < ue) {
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
                    if (j < ue) {
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
                            const uint2 mq = reinterpret_cast<const uint2 *>(hi + p.nb)[j];
                            const uint4 l = lo[j], h = hi[j];
                            const float d8 = __uint_as_float(mq.x);
                            acc = fmaf((float)q4_block_dot(w[u], l, h, (int)mq.y), __half2float(sc[u]) * d8, acc);
                            if (GATED) acc2 = fmaf((float)q4_block_dot(w2[u], l, h, (int)mq.y), __half2float(sc2[u]) * d8, acc2);
                        }
                    }
                }
            }
            acc = warp_sum(acc);
            if (GATED) acc2 = warp_sum(acc2);
            if (lane == 0) {
                s_part[(rl * ROWS_WARPS + wid) * NM] += acc;
                if (GATED) s_part[(rl * ROWS_WARPS + wid) * NM + 1] += acc2;
            }
            cur += (unsigned)(ue - ub);
        }
    }
    __syncthreads();
    PI_TL_MARK(2);
    cl_wait();                                                       // every CTA of the cluster runs: its shared memory may be written
    for (int t = tid; t < mj; t += ROWS_THREADS) {
        float up = 0.f, gt = 0.f;
#pragma unroll
        for (int w = 0; w < ROWS_WARPS; w++) {                      // warps that held no piece of the row left 0
            up += s_part[(t * ROWS_WARPS + w) * NM];
            if (GATED) gt += s_part[(t * ROWS_WARPS + w) * NM + 1];
        }
        const int r = s_myrow[t];
        float o = up;
        if (GATED) o = fmaxf(gt, 0.f) * up;
        if (p.bias) o += p.bias[r];
        if (p.relu) o = fmaxf(o, 0.f);
        if (p.h_out) p.h_out[r] = o;
        for (int q = 0; q < CS; q++) {
            cl_store_u32(s_h + i0 + t, (unsigned)q, __float_as_uint(o));
            cl_store_u32(s_rowc + i0 + t, (unsigned)q, (uint32_t)r);
        }
    }
    cl_arrive();
    cl_wait();                                                       // the cluster's activations are in every CTA's shared memory
    PI_TL_MARK(3);

    // ================================================================= coefficients; rows whose coefficient is not zero
    // Coefficient = what the CPU path multiplies the row by: FP16(h) for FP16 rows; for Q4_0 the int8 quant of h within its
    // block of 32 neurons times that block's FP16 scale (ggml.c:14575-14581, quantize_row_q8_0).  Inactive neurons of the
    // block count as 0, so the largest |h| is taken over the block's active rows, which are neighbours in rank order.
    if (tid == 0) s_cnt = 0;
    __syncthreads();
    for (int t0 = 0; t0 < m; t0 += ROWS_THREADS) {
        const int t = t0 + tid;
        int r = -1; float c = 0.f;
        if (t < m) {
            r = s_rowc[t];
            const float hv = s_h[t];
            if (WT == PI_TYPE_F16) {
                c = round_f16(hv);
            } else {
                const int ch = r >> 5;
                const int f = s_pref[ch] - r0, cnt = __popc(s_mask[ch]);
                float amax = 0.f;
                for (int i = 0; i < cnt; i++) { const int k = f + i; if (k >= 0 && k < m) amax = fmaxf(amax, fabsf(s_h[k])); }
                const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
                c = (float)__float2int_rn(hv * id) * round_f16(amax / 127.0f);
            }
        }
        const bool keep = r >= 0 && c != 0.f;                       // keep the order: ballot inside the warp, warp offsets through shared memory
        const unsigned bal = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) s_warp[wid] = __popc(bal);
        __syncthreads();
        int off = s_cnt;
        for (int w = 0; w < wid; w++) off += s_warp[w];
        if (keep) { const int o = off + __popc(bal & ((1u << lane) - 1u)); s_row2[o] = r; s_coef[o] = c; }
        __syncthreads();
        if (tid == 0) { int tot = 0; for (int w = 0; w < ROWS_WARPS; w++) tot += s_warp[w]; s_cnt += tot; }
        __syncthreads();
    }
    const int m2 = s_cnt;
    PI_TL_MARK(4);

    // ================================================================= axpy over the slices j, j + CS, ... of down_t
    // NS slices at a time (their loads travel together).  Warp w takes entries w, w + 16, ...; a lane owns 32 columns of a slice:
    //   Q4_0: block `slice * 32 + lane` (sum index = column inside the block);
    //   FP16: 8 columns at 8 * lane of each of the slice's four 256-column quarters (sum index = 8 * quarter + e).
    constexpr int UA = (WT == PI_TYPE_F16 ? 4 : 8) / NS;            // rows in flight per warp
    const int n_slices = (p.ncols + SLICE - 1) / SLICE;
    for (int slice0 = cj; slice0 < n_slices; slice0 += CS * NS) {
        unsigned long long acc[NS][16];
        float corr[NS];
        int unit0[NS];
#pragma unroll
        for (int s = 0; s < NS; s++) {
#pragma unroll
            for (int j = 0; j < 16; j++) acc[s][j] = 0ull;
            corr[s] = 0.f;
            const int slice = slice0 + s * CS;                       // a slice beyond the last one loads nothing (unit0 >= units)
            unit0[s] = WT == PI_TYPE_F16 ? slice * (SLICE / 8) + lane : slice * 32 + lane;
        }
        for (int e0 = wid; e0 < m2; e0 += ROWS_WARPS * UA) {
            if (WT == PI_TYPE_Q4_0) {
                uint4 q[UA][NS]; __half d4[UA][NS]; float c[UA];
#pragma unroll
                for (int u = 0; u < UA; u++) {
                    const int i = e0 + u * ROWS_WARPS;
                    c[u] = 0.f;
                    const uint8_t * row = i < m2 ? p.Wdown + (size_t)s_row2[i] * p.row_bytes : nullptr;
                    if (i < m2) c[u] = s_coef[i];
#pragma unroll
                    for (int s = 0; s < NS; s++) {
                        q[u][s] = make_uint4(0u, 0u, 0u, 0u); d4[u][s] = __ushort_as_half((unsigned short)0);
                        if (i < m2 && unit0[s] < units) {
                            q[u][s] = ldg_stream(reinterpret_cast<const uint4 *>(row) + unit0[s]);
                            d4[u][s] = __ldg(reinterpret_cast<const __half *>(row + (size_t)p.nb * 16) + unit0[s]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < UA; u++) {
#pragma unroll
                    for (int s = 0; s < NS; s++) {
                        // nibble q -> the float 16 + q with one byte permute (q lands in mantissa bits 19..22 under the exponent
                        // of 16); (q - 8) * sc = (16 + q) * sc - 24 * sc, and the second term is summed once per row instead of
                        // once per weight (costs under 2 bits of the FP32 accumulator)
                        const float sc = c[u] * __half2float(d4[u][s]);
                        corr[s] += sc;
                        const unsigned long long sc2 = pack2(sc, sc);
                        const uint32_t wds[4] = {q[u][s].x, q[u][s].y, q[u][s].z, q[u][s].w};
#pragma unroll
                        for (int wi = 0; wi < 4; wi++) {
                            const uint32_t lo = ((wds[wi] << 3) & 0x78787878u) | 0x80808080u;
                            const uint32_t hi = ((wds[wi] >> 1) & 0x78787878u) | 0x80808080u;
                            const unsigned long long l01 = (unsigned long long)__byte_perm(lo, 0x41000000u, 0x7044u) | ((unsigned long long)__byte_perm(lo, 0x41000000u, 0x7144u) << 32);
                            const unsigned long long l23 = (unsigned long long)__byte_perm(lo, 0x41000000u, 0x7244u) | ((unsigned long long)__byte_perm(lo, 0x41000000u, 0x7344u) << 32);
                            const unsigned long long h01 = (unsigned long long)__byte_perm(hi, 0x41000000u, 0x7044u) | ((unsigned long long)__byte_perm(hi, 0x41000000u, 0x7144u) << 32);
                            const unsigned long long h23 = (unsigned long long)__byte_perm(hi, 0x41000000u, 0x7244u) | ((unsigned long long)__byte_perm(hi, 0x41000000u, 0x7344u) << 32);
                            ffma2(acc[s][wi * 2], l01, sc2); ffma2(acc[s][wi * 2 + 1], l23, sc2);
                            ffma2(acc[s][8 + wi * 2], h01, sc2); ffma2(acc[s][8 + wi * 2 + 1], h23, sc2);
                        }
                    }
                }
            } else {
                uint4 w[UA][NS][4]; float c[UA];
#pragma unroll
                for (int u = 0; u < UA; u++) {
                    const int i = e0 + u * ROWS_WARPS;
                    c[u] = 0.f;
                    const uint4 * row = i < m2 ? reinterpret_cast<const uint4 *>(p.Wdown + (size_t)s_row2[i] * p.row_bytes) : nullptr;
                    if (i < m2) c[u] = s_coef[i];
#pragma unroll
                    for (int s = 0; s < NS; s++) {
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            w[u][s][k] = make_uint4(0u, 0u, 0u, 0u);
                            if (i < m2 && unit0[s] + k * 32 < units) w[u][s][k] = ldg_stream(row + unit0[s] + k * 32);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < UA; u++) {
                    const unsigned long long c2 = pack2(c[u], c[u]);
#pragma unroll
                    for (int s = 0; s < NS; s++) {
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const float2 f0 = h2f(w[u][s][k].x), f1 = h2f(w[u][s][k].y), f2 = h2f(w[u][s][k].z), f3 = h2f(w[u][s][k].w);
                            ffma2(acc[s][k * 4 + 0], pack2(f0.x, f0.y), c2); ffma2(acc[s][k * 4 + 1], pack2(f1.x, f1.y), c2);
                            ffma2(acc[s][k * 4 + 2], pack2(f2.x, f2.y), c2); ffma2(acc[s][k * 4 + 3], pack2(f3.x, f3.y), c2);
                        }
                    }
                }
            }
        }
        // warps are added in warp order through shared memory (sum index a of lane l at a * 33 + l: no bank conflicts)
        __syncthreads();                                             // the region's previous content is dead for every warp
#pragma unroll
        for (int s = 0; s < NS; s++) {
            float * mine = s_red + ((size_t)s * ROWS_WARPS + wid) * (32 * 33);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                float a0 = lo_f(acc[s][j]), a1 = hi_f(acc[s][j]);
                if (WT == PI_TYPE_Q4_0) { a0 = fmaf(-24.0f, corr[s], a0); a1 = fmaf(-24.0f, corr[s], a1); }
                mine[(2 * j) * 33 + lane] = a0;
                mine[(2 * j + 1) * 33 + lane] = a1;
            }
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < NS; s++) {
            const int slice = slice0 + s * CS;
            if (slice >= n_slices) break;
            float * out = p.partial + (size_t)cluster * p.ncols + (size_t)slice * SLICE;
            for (int cidx = tid; cidx < SLICE; cidx += ROWS_THREADS) {
                if ((size_t)slice * SLICE + cidx >= (size_t)p.ncols) break;
                int a, l;
                if (WT == PI_TYPE_Q4_0) { l = cidx >> 5; a = cidx & 31; }
                else                    { const int q = cidx >> 8; l = (cidx & 255) >> 3; a = q * 8 + (cidx & 7); }
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < ROWS_WARPS; w++) v += s_red[((size_t)s * ROWS_WARPS + w) * (32 * 33) + a * 33 + l];
                out[cidx] = v;
            }
        }
    }
    PI_TL_MARK(5);
}

// ---------------------------------------------------------------------------------------------- launch
namespace {

struct FfnPlan { bool ok = false; int cs = 0, ns = 0, n_clusters = 0, cap = 0, cap_cta = 0; size_t smem = 0; };

size_t ffn_smem(int wtype, int64_t ncols, int n_chunks, int cap, int cap_cta, bool gated, int ns) {
    const size_t x_bytes = wtype == PI_TYPE_F16 ? (size_t)ncols * 2 : (size_t)(ncols / QK) * 40;
    const size_t lists = up128((size_t)(2 * n_chunks + 1) * 4 + (size_t)cap * 16 + (size_t)cap_cta * 4);
    const size_t gather = up128(x_bytes) + (size_t)cap_cta * ROWS_WARPS * (gated ? 2 : 1) * 4;
    const size_t red = (size_t)ns * ROWS_WARPS * 32 * 33 * 4;
    return lists + (gather > red ? gather : red) + 128;
}

// the plan for cluster size cs with this kernel instance: as many clusters as can be resident at once (so no cluster waits
// for another one to finish), capped by the partial vectors the caller has room for
template <int WT, bool GATED, int U, int NS>
bool ffn_plan_cs(const FfnRowsArgs & a, int cs, FfnPlan & pl) {
    auto kern = k_ffn_rows<WT, GATED, U, NS>;
    static bool attr_done[16] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) { cudaGetLastError(); return false; }
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) cudaGetLastError();   // clusters of 16
        attr_done[dev] = true;
    }
    const int n_chunks = (int)((a.nrows + 31) / 32);
    int nc = sm_count() / cs;
    if (nc > a.n_groups) nc = a.n_groups;
    for (int pass = 0; pass < 2 && nc >= 1; pass++) {
        // room for the rows of a cluster: its share of ALL rows (every neuron active) plus the slack of whole mask words
        const int cap = (int)(((a.nrows + nc - 1) / nc + 40 + 7) / 8 * 8);
        const int cap_cta = (cap + cs - 1) / cs + 1;
        const size_t smem = ffn_smem(WT, a.ncols, n_chunks, cap, cap_cta, GATED, NS);
        if (smem > 200 * 1024) return false;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(nc * cs); cfg.blockDim = dim3(ROWS_THREADS); cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int max_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
        if (max_clusters < 1) return false;
        if (max_clusters < nc) { nc = max_clusters; continue; }                  // once more with the smaller count (cap grows)
        pl.ok = true; pl.cs = cs; pl.ns = NS; pl.n_clusters = nc; pl.cap = cap; pl.cap_cta = cap_cta; pl.smem = smem;
        return true;
    }
    return false;
}

template <int WT, bool GATED, int U, int NS>
int ffn_go(const FfnRowsP & p0, const FfnPlan & pl, bool pdl, cudaStream_t st) {
    FfnRowsP p = p0;
    p.n_clusters = pl.n_clusters; p.cap = pl.cap; p.cap_cta = pl.cap_cta;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.n_clusters * pl.cs); cfg.blockDim = dim3(ROWS_THREADS); cfg.dynamicSmemBytes = pl.smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 2 : 1;
    PI_CUDA(cudaLaunchKernelEx(&cfg, k_ffn_rows<WT, GATED, U, NS>, p));
    return PI_OK;
}

template <int WT, bool GATED>
int ffn_launch(const FfnRowsP & p, const FfnRowsArgs & a, int * groups_used, cudaStream_t st, bool plan_only) {
    constexpr int U = 8;                                            // 128-bit loads per matrix in flight per lane
    // one plan per device and shape (PI_FFN_CS forces a cluster size)
    struct Key { int dev; int64_t nrows, ncols; int groups; FfnPlan pl; };
    static Key cache[8];
    static int n_cache = 0;
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    FfnPlan pl;
    bool found = false;
    for (int i = 0; i < n_cache; i++)
        if (cache[i].dev == dev && cache[i].nrows == a.nrows && cache[i].ncols == a.ncols && cache[i].groups == a.n_groups) { pl = cache[i].pl; found = true; }
    if (!found) {
        static int forced = -1;
        if (forced < 0) { const char * v = getenv("PI_FFN_CS"); forced = v ? atoi(v) : 0; }
        const int n_slices = (int)((a.ncols + SLICE - 1) / SLICE);
        for (int cs = 16; cs >= 2; cs--) {
            if (forced ? cs != forced : (cs != 8 && cs != 4 && cs != 2)) continue;     // other sizes only on request
            FfnPlan c;
            const bool two = (n_slices + cs - 1) / cs >= 2;
            const bool ok = two ? ffn_plan_cs<WT, GATED, U, 2>(a, cs, c) : ffn_plan_cs<WT, GATED, U, 1>(a, cs, c);
            // The largest cluster that can be launched wins although it keeps fewer SMs busy (15 x 8 = 120 of 148 on a B200
            // against 33 x 4 = 132): it leaves half the partial vectors, which the norm after this kernel reads in one pass
            // instead of two (measured per step: 6.11 ms against 6.25 ms).
            if (ok && !pl.ok) pl = c;
        }
        if (getenv("PI_FFN_VERBOSE"))
            fprintf(stderr, "sparse FFN kernel plan: rows %lld cols %lld -> %s, cluster size %d, %d clusters, %d slices at a time, %zu bytes of shared memory\n",
                    (long long)a.nrows, (long long)a.ncols, pl.ok ? "one launch" : "not eligible", pl.cs, pl.n_clusters, pl.ns, pl.smem);
        if (n_cache < 8) { cache[n_cache].dev = dev; cache[n_cache].nrows = a.nrows; cache[n_cache].ncols = a.ncols; cache[n_cache].groups = a.n_groups; cache[n_cache].pl = pl; n_cache++; }
    }
    if (!pl.ok) return PI_ERR_UNSUPPORTED;
    if (groups_used) *groups_used = pl.n_clusters;
    if (plan_only) return PI_OK;
    return pl.ns == 2 ? ffn_go<WT, GATED, U, 2>(p, pl, a.pdl, st) : ffn_go<WT, GATED, U, 1>(p, pl, a.pdl, st);
}

}  // namespace

static int ffn_rows_do(const FfnRowsArgs & a, cudaStream_t st, int * groups_used, bool plan_only) {
    static int enabled = -1;                                        // PI_FFN_FUSED=0: the two separate kernels (diagnostic)
    if (enabled < 0) { const char * v = getenv("PI_FFN_FUSED"); enabled = !(v && v[0] == '0'); }
    if (!enabled || !a.up || !a.down_t || !rows_eligible(a.wtype, a.nrows, a.ncols)) return PI_ERR_UNSUPPORTED;
    if (!plan_only && (!a.masks || !a.partial)) return PI_ERR_UNSUPPORTED;
    FfnRowsP p;
    p.Wup = (const uint8_t *)a.up; p.Wgate = (const uint8_t *)a.gate; p.Wdown = (const uint8_t *)a.down_t;
    p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols); p.nrows = (int)a.nrows; p.ncols = (int)a.ncols;
    p.nb = (int)(a.ncols / QK); p.n_chunks = (int)((a.nrows + 31) / 32);
    p.x = a.x; p.masks = a.masks; p.bias = a.bias; p.relu = a.relu; p.h_out = a.h; p.partial = a.partial; p.rows_total = a.rows_total;
    p.n_clusters = 0; p.cap = 0; p.cap_cta = 0;
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    if (a.gate) return q4 ? ffn_launch<PI_TYPE_Q4_0, true>(p, a, groups_used, st, plan_only) : ffn_launch<PI_TYPE_F16, true>(p, a, groups_used, st, plan_only);
    return q4 ? ffn_launch<PI_TYPE_Q4_0, false>(p, a, groups_used, st, plan_only) : ffn_launch<PI_TYPE_F16, false>(p, a, groups_used, st, plan_only);
}

int launch_ffn_rows(const FfnRowsArgs & a, cudaStream_t st, int * groups_used) { return ffn_rows_do(a, st, groups_used, false); }

// does launch_ffn_rows take this shape on the current device (weights and n_groups as they will be passed)?
bool ffn_rows_eligible(const FfnRowsArgs & a) { return ffn_rows_do(a, nullptr, nullptr, true) == PI_OK; }

}  // namespace pi
