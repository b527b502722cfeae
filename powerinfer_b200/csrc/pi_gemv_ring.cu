// Batch-1 mat-vec with the weights streamed through a shared-memory ring by the bulk-copy engine.
//
// One persistent CTA per SM.  A stage of the ring holds R weight rows (R consecutive rows of a dense matrix: ONE bulk
// copy; R rows named by the active list for ggml_mul_mat_idx: R copies, plus the R gate rows when the gate matrix rides
// along).  An mbarrier per stage counts the bytes that land; the 8 consumer warps then read the rows from shared
// memory (conflict-free 128-bit reads), so the bytes in flight per SM are set by the ring size (~190 KB), not by
// registers or occupancy, and DRAM sees large sequential requests.
// Weights never depend on the previous kernel, so with programmatic dependent launch the first ring fill of a dense
// matrix is issued BEFORE griddepcontrol.wait: it overlaps the tail of whatever produced the activation.
// cp.async.bulk here is the plain (non-tensor, non-multicast) form; sources are this GPU's own memory.
// Every mbarrier wait is bounded: on expiry the CTA sets bit 2 of *status, stops, and drains its copies.
#include "pi_common.cuh"

#include <cstdlib>

namespace pi {

static constexpr int QK = 32;
static constexpr int RING_THREADS = 256;
static constexpr int RING_WARPS = 8;
static constexpr int RING_MAX_ITEMS = 1024;            // list entries one CTA may own
static constexpr int RING_MAX_VEC = 128;               // row vectors in one stage (rows x matrices)


struct RingP {
    const uint8_t * W; const uint8_t * W2;
    int64_t row_bytes; int nrows; int ncols; int nb;
    Act x;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; float threshold;
    const float * bias; int relu;
    float * dst; __half * dst16;
    uint32_t * masks_out; float masks_threshold;
    int pre;
    unsigned int * status;
    int R, split, stages, max_items; size_t stage_bytes;
};

__device__ __forceinline__ int r_block_dot(const uint4 q, const uint4 lo, const uint4 hi, int s8) {
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

// dot of the staged row (shared memory) with the staged activation over 16-byte units [u_lo, u_hi): FP16: 8 columns per
// unit; Q4_0: one 32-column block per unit
template <int WT>
__device__ __forceinline__ float ring_row_dot(const unsigned char * row, int u_lo, int u_hi, int nb, const unsigned char * xs, int lane) {
    float acc0 = 0.f, acc1 = 0.f;
    if (WT == PI_TYPE_F16) {
        const uint4 * w = reinterpret_cast<const uint4 *>(row);
        const uint4 * x = reinterpret_cast<const uint4 *>(xs);
        for (int u = u_lo + lane; u < u_hi; u += 64) {
            {
                const uint4 wv = w[u], xv = x[u];
                const float2 w0 = h2f(wv.x), w1 = h2f(wv.y), w2 = h2f(wv.z), w3 = h2f(wv.w);
                const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
                acc0 = fmaf(w0.x, x0.x, acc0); acc0 = fmaf(w0.y, x0.y, acc0); acc0 = fmaf(w1.x, x1.x, acc0); acc0 = fmaf(w1.y, x1.y, acc0);
                acc0 = fmaf(w2.x, x2.x, acc0); acc0 = fmaf(w2.y, x2.y, acc0); acc0 = fmaf(w3.x, x3.x, acc0); acc0 = fmaf(w3.y, x3.y, acc0);
            }
            if (u + 32 < u_hi) {
                const uint4 wv = w[u + 32], xv = x[u + 32];
                const float2 w0 = h2f(wv.x), w1 = h2f(wv.y), w2 = h2f(wv.z), w3 = h2f(wv.w);
                const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
                acc1 = fmaf(w0.x, x0.x, acc1); acc1 = fmaf(w0.y, x0.y, acc1); acc1 = fmaf(w1.x, x1.x, acc1); acc1 = fmaf(w1.y, x1.y, acc1);
                acc1 = fmaf(w2.x, x2.x, acc1); acc1 = fmaf(w2.y, x2.y, acc1); acc1 = fmaf(w3.x, x3.x, acc1); acc1 = fmaf(w3.y, x3.y, acc1);
            }
        }
    } else {
        const uint4 * q = reinterpret_cast<const uint4 *>(row);
        const __half * sc = reinterpret_cast<const __half *>(row + (size_t)nb * 16);
        const uint4 * lo = reinterpret_cast<const uint4 *>(xs);
        const uint4 * hi = lo + nb;
        const uint2 * ds = reinterpret_cast<const uint2 *>(hi + nb);        // {scale as float bits, int8 sum} per block
        for (int b = u_lo + lane; b < u_hi; b += 64) {
            const uint2 m = ds[b];
            acc0 = fmaf((float)r_block_dot(q[b], lo[b], hi[b], (int)m.y), __half2float(sc[b]) * __uint_as_float(m.x), acc0);
            if (b + 32 < u_hi) {
                const int c = b + 32;
                const uint2 m2 = ds[c];
                acc1 = fmaf((float)r_block_dot(q[c], lo[c], hi[c], (int)m2.y), __half2float(sc[c]) * __uint_as_float(m2.x), acc1);
            }
        }
    }
    return acc0 + acc1;
}

// RW staged vectors (consecutive, row_bytes apart) against the staged activation over units [u_lo, u_hi): the
// activation unit is read from shared memory and converted once and used for all RW rows, and the RW sums are
// independent dependency chains.
template <int WT, int RW>
__device__ __forceinline__ void ring_dot_rows(const unsigned char * base, size_t row_bytes, int u_lo, int u_hi, int nb,
                                              const unsigned char * xs, int lane, float (&acc)[RW]) {
#pragma unroll
    for (int r = 0; r < RW; r++) acc[r] = 0.f;
    if (WT == PI_TYPE_F16) {
        const uint4 * x = reinterpret_cast<const uint4 *>(xs);
#pragma unroll 2
        for (int u = u_lo + lane; u < u_hi; u += 32) {
            const uint4 xv = x[u];
            const float2 x0 = h2f(xv.x), x1 = h2f(xv.y), x2 = h2f(xv.z), x3 = h2f(xv.w);
#pragma unroll
            for (int r = 0; r < RW; r++) {
                const uint4 wv = reinterpret_cast<const uint4 *>(base + (size_t)r * row_bytes)[u];
                const float2 w0 = h2f(wv.x), w1 = h2f(wv.y), w2 = h2f(wv.z), w3 = h2f(wv.w);
                float a = acc[r];
                a = fmaf(w0.x, x0.x, a); a = fmaf(w0.y, x0.y, a); a = fmaf(w1.x, x1.x, a); a = fmaf(w1.y, x1.y, a);
                a = fmaf(w2.x, x2.x, a); a = fmaf(w2.y, x2.y, a); a = fmaf(w3.x, x3.x, a); a = fmaf(w3.y, x3.y, a);
                acc[r] = a;
            }
        }
    } else {
        const uint4 * lo = reinterpret_cast<const uint4 *>(xs);
        const uint4 * hi = lo + nb;
        const uint2 * ds = reinterpret_cast<const uint2 *>(hi + nb);        // {scale as float bits, int8 sum} per block
#pragma unroll 2
        for (int b = u_lo + lane; b < u_hi; b += 32) {
            const uint4 l = lo[b], h = hi[b];
            const uint2 m = ds[b];
            const float d8 = __uint_as_float(m.x);
#pragma unroll
            for (int r = 0; r < RW; r++) {
                const unsigned char * row = base + (size_t)r * row_bytes;
                const uint4 q = reinterpret_cast<const uint4 *>(row)[b];
                const float d4 = __half2float(reinterpret_cast<const __half *>(row + (size_t)nb * 16)[b]);
                acc[r] = fmaf((float)r_block_dot(q, l, h, (int)m.y), d4 * d8, acc[r]);
            }
        }
    }
}

template <int WT, bool SPARSE, bool GATED, int RW>
__global__ void __launch_bounds__(RING_THREADS) k_gemv_ring(const RingP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float s_part[2][RING_MAX_VEC][RING_WARPS];          // [stage parity][vector of the stage][column part]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages, R = p.R, split = p.split;
    const int NM = GATED ? 2 : 1;                                  // matrices riding in one stage

    // shared-memory map: [S] mbarriers | item list | staged activation | ring
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    int * items = reinterpret_cast<int *>(smem + 8 * 32);
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * xs = smem + (((size_t)8 * 32 + (size_t)4 * p.max_items + 127) & ~(size_t)127);
    unsigned char * ring = xs + ((x_bytes + 127) & ~(size_t)127);

    pdl_launch();                                                   // let the next kernel become resident and prefetch
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // stage st of this CTA covers items [ (cta + st*G) * R, +R ) of the row / list sequence
    int n_items, n_stages;
    auto stage_first = [&](int st) { return (cta + st * G) * R; };
    auto issue = [&](int st) {                                       // all lanes of warp 0
        const int s = st % S;
        const int first = stage_first(st);
        const int n = min(R, n_items - first);
        unsigned char * dstp = ring + (size_t)s * p.stage_bytes;
        if (!SPARSE) {
            if (lane == 0) {
                mbar_expect_tx(full + s, (unsigned)(n * p.row_bytes));
                bulk_g2s(dstp, p.W + (size_t)first * p.row_bytes, (unsigned)(n * p.row_bytes), full + s);
            }
        } else {
            // the phase cannot complete before the arrive below, whatever the order in which the lanes' copies land
            if (lane == 0) mbar_expect_tx(full + s, (unsigned)(n * NM * p.row_bytes));
            for (int k = lane; k < n; k += 32) {
                const int r = items[st * R + k];
                bulk_g2s(dstp + (size_t)k * p.row_bytes, p.W + (size_t)r * p.row_bytes, (unsigned)p.row_bytes, full + s);
                if (GATED) bulk_g2s(dstp + (size_t)(R + k) * p.row_bytes, p.W2 + (size_t)r * p.row_bytes, (unsigned)p.row_bytes, full + s);
            }
        }
    };

    if (!SPARSE) {
        // dense: the rows are known now; fill the ring before waiting for the producer of the activation
        n_items = p.nrows;
        const int total_stages = (n_items + R - 1) / R;
        n_stages = cta < total_stages ? (total_stages - cta + G - 1) / G : 0;
        if (warp == 0) for (int st = 0; st < S && st < n_stages; st++) issue(st);
    }
    pdl_wait();
    if (SPARSE) {
        n_items = min(*p.count, p.nrows);
        const int total_stages = (n_items + R - 1) / R;
        n_stages = cta < total_stages ? (total_stages - cta + G - 1) / G : 0;
        n_stages = min(n_stages, p.max_items / R);
        for (int i = tid; i < n_stages * R; i += RING_THREADS) {
            const int it = stage_first(i / R) + (i % R);
            int r = it < n_items ? p.list[it] : 0;
            items[i] = (unsigned)r < (unsigned)p.nrows ? r : 0;
        }
        __syncthreads();
        if (warp == 0) for (int st = 0; st < S && st < n_stages; st++) issue(st);
    }
    // ---- stage the activation
    if (WT == PI_TYPE_F16) {
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dstx = reinterpret_cast<uint4 *>(xs);
        for (int i = tid; i < p.ncols / 8; i += RING_THREADS) dstx[i] = src[i];
    } else {
        uint4 * lo = reinterpret_cast<uint4 *>(xs);
        uint4 * hi = lo + p.nb;
        uint2 * ds = reinterpret_cast<uint2 *>(hi + p.nb);
        for (int i = tid; i < p.nb; i += RING_THREADS) {
            lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i];
            ds[i] = make_uint2(__float_as_uint(p.x.d[i]), (unsigned)p.x.s[i]);
        }
    }
    __syncthreads();

    // A stage holds NV = R * NM vectors (the R gate rows after the R up rows).  RW consecutive vectors form a group that
    // one warp reads together; `split` warps share a group, each taking 1/split of the columns.  Partial sums go through
    // shared memory and are added in part order by the thread that owns the row.
    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;       // 16-byte units per row
    const int per = units / split;
    const int NV = R * NM, groups = NV / RW;
    bool dead = false;                                              // warp-uniform
    for (int st = 0; st < n_stages; st++) {
        const int s = st % S;
        const unsigned parity = (unsigned)(st / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            dead = __any_sync(0xffffffffu, gave_up) != 0;            // the whole warp agrees, so no shuffle runs half-populated
            if (dead && lane == 0) atomicOr(p.status, 4u);
        }
        const unsigned char * base = ring + (size_t)s * p.stage_bytes;
        const int first = stage_first(st);
        const int n = min(R, n_items - first);
        float (*part_sums)[RING_WARPS] = s_part[st & 1];
        for (int g = warp / split; g < groups; g += RING_WARPS / split) {
            const int part = warp % split;
            float acc[RW];
            if (!dead) ring_dot_rows<WT, RW>(base + (size_t)g * RW * p.row_bytes, (size_t)p.row_bytes, part * per, (part + 1) * per, p.nb, xs, lane, acc);
#pragma unroll
            for (int r = 0; r < RW; r++) {
                const float v = dead ? 0.f : warp_sum(acc[r]);
                if (lane == 0) part_sums[g * RW + r][part] = v;
            }
        }
        __syncthreads();                                             // sums visible; every warp is done with stage s
        if (warp == 0 && !dead && st + S < n_stages) issue(st + S);
        if (tid >= 32 && tid - 32 < n) {                             // warps 1..: warp 0 is busy refilling the stage
            const int k = tid - 32;
            float v = part_sums[k][0], v2 = 0.f;
            for (int q = 1; q < split; q++) v += part_sums[k][q];
            if (GATED) { v2 = part_sums[R + k][0]; for (int q = 1; q < split; q++) v2 += part_sums[R + k][q]; }
            const int r = SPARSE ? items[st * R + k] : first + k;
            const int64_t g = SPARSE && p.bucket ? p.bucket[r] : r;
            // batch 1: a listed row is an active row (the list was made from the same logits and threshold)
            float o = v;
            if (GATED) o = fmaxf(v2, 0.f) * v;
            if (p.bias) o += p.bias[g];
            if (p.relu) o = fmaxf(o, 0.f);
            if (p.dst)   p.dst[g] = o;
            if (p.dst16) p.dst16[g] = __float2half_rn(o);
        }
    }
    if (__syncthreads_or(dead) && tid == 0) {                       // do not exit with copies still landing in shared memory
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
}

// Dense matrices whose stage holds at least one row per warp (R >= 8): every warp owns whole rows of the stage, so nothing
// is exchanged between warps, and the stage is handed back through a second ("empty") mbarrier on which each warp arrives
// when it is done: only warp 0, which refills the stage, waits for the others; the rest go straight on to the next stage.
// Halving the stage size in the kernel above costs 1.7 ms per 70B-shape token: its per-stage block barrier, shared-memory
// exchange of partial sums and result hand-off are a fixed cost comparable to the stage's streaming time.

template <int WT>
__global__ void __launch_bounds__(RING_THREADS) k_gemv_ring_w(const RingP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages, R = p.R;
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);           // [S] at byte 0, [S] "empty" at byte 128 (S <= 8)
    uint64_t * empty = reinterpret_cast<uint64_t *>(smem + 128);
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * xs = smem + 256;
    unsigned char * ring = xs + ((x_bytes + 127) & ~(size_t)127);

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full + s, 1); mbar_init(empty + s, RING_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const int n_items = p.nrows;
    const int total_stages = (n_items + R - 1) / R;
    const int n_stages = cta < total_stages ? (total_stages - cta + G - 1) / G : 0;
    auto stage_first = [&](int st) { return (cta + st * G) * R; };
    auto issue = [&](int st) {                                       // lane 0 of warp 0
        const int s = st % S, first = stage_first(st), n = min(R, n_items - first);
        mbar_expect_tx(full + s, (unsigned)(n * p.row_bytes));
        bulk_g2s(ring + (size_t)s * p.stage_bytes, p.W + (size_t)first * p.row_bytes, (unsigned)(n * p.row_bytes), full + s);
    };
    const int pre = p.pre < 0 ? S : min(p.pre, S);
    if (tid == 0) for (int st = 0; st < pre && st < n_stages; st++) issue(st);   // weights need no producer: before the wait
    pdl_wait();
    if (tid == 0) for (int st = pre; st < S && st < n_stages; st++) issue(st);
    if (WT == PI_TYPE_F16) {
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dstx = reinterpret_cast<uint4 *>(xs);
        for (int i = tid; i < p.ncols / 8; i += RING_THREADS) dstx[i] = src[i];
    } else {
        uint4 * lo = reinterpret_cast<uint4 *>(xs);
        uint4 * hi = lo + p.nb;
        uint2 * ds = reinterpret_cast<uint2 *>(hi + p.nb);
        for (int i = tid; i < p.nb; i += RING_THREADS) {
            lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i];
            ds[i] = make_uint2(__float_as_uint(p.x.d[i]), (unsigned)p.x.s[i]);
        }
    }
    __syncthreads();

    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;
    const int rpw = R / RING_WARPS;                                 // rows of a stage per warp (1, 2, 4 or 8), consecutive
    bool dead = false;                                              // warp-uniform
    auto store = [&](int r, float o) -> unsigned {
        if (p.bias) o += p.bias[r];
        if (p.relu) o = fmaxf(o, 0.f);
        if (p.dst)   p.dst[r] = o;
        if (p.dst16) p.dst16[r] = __float2half_rn(o);
        return (o < p.masks_threshold) ? 0u : 1u;                  // a NaN counts as active, as where the reference skips on `<`
    };
    // activity masks of the result (masks_out): lane 0 of every warp leaves the bits of its rows of a stage in a byte of
    // shared memory before it hands the stage back; warp 0, which waits for all eight hand-backs anyway, joins them and
    // writes the stage's R bits: no atomics, nothing to clear beforehand
    unsigned char * s_bits = smem + 192;                            // [S][RING_WARPS]
    for (int st = 0; st < n_stages; st++) {
        const int s = st % S;
        const unsigned parity = (unsigned)(st / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            dead = __any_sync(0xffffffffu, gave_up) != 0;
            if (dead && lane == 0) atomicOr(p.status, 4u);
        }
        const unsigned char * base = ring + (size_t)s * p.stage_bytes;
        const int first = stage_first(st);
        const int n = min(R, n_items - first);
        unsigned bits = 0u;
        if (!dead) {
            int k = warp * rpw;
            const int k_end = min(k + rpw, n);
            for (; k + 2 <= k_end; k += 2) {
                float acc[2];
                ring_dot_rows<WT, 2>(base + (size_t)k * p.row_bytes, (size_t)p.row_bytes, 0, units, p.nb, xs, lane, acc);
                const float v0 = warp_sum(acc[0]), v1 = warp_sum(acc[1]);
                if (lane == 0) { bits |= store(first + k, v0) << (k - warp * rpw); bits |= store(first + k + 1, v1) << (k + 1 - warp * rpw); }
            }
            if (k < k_end) {
                float acc[1];
                ring_dot_rows<WT, 1>(base + (size_t)k * p.row_bytes, (size_t)p.row_bytes, 0, units, p.nb, xs, lane, acc);
                const float v0 = warp_sum(acc[0]);
                if (lane == 0) bits |= store(first + k, v0) << (k - warp * rpw);
            }
        }
        if (p.masks_out && lane == 0) s_bits[s * RING_WARPS + warp] = (unsigned char)bits;
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);                     // this warp is done with stage s (also when it gave up)
        if (warp == 0 && (st + S < n_stages || p.masks_out)) {       // refill / masks: wait (bounded) until every warp has arrived
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(empty + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            if (gave_up) { if (lane == 0) atomicOr(p.status, 4u); }
            else if (lane == 0 && !dead) {
                if (p.masks_out) {
                    unsigned long long m = 0ull;
                    for (int w = 0; w < RING_WARPS; w++) m |= (unsigned long long)s_bits[s * RING_WARPS + w] << (w * rpw);
                    unsigned char * mo = reinterpret_cast<unsigned char *>(p.masks_out) + first / 8;      // first % R == 0
                    if (R == 8)       *mo = (unsigned char)m;
                    else if (R == 16) *reinterpret_cast<unsigned short *>(mo) = (unsigned short)m;
                    else if (R == 32) *reinterpret_cast<unsigned int *>(mo) = (unsigned int)m;
                    else              *reinterpret_cast<unsigned long long *>(mo) = m;
                }
                if (st + S < n_stages) issue(st + S);
            }
        }
    }
    if (__syncthreads_or(dead) && tid == 0) {                       // do not exit with copies still landing in shared memory
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
}

// The same hand-off for stages of fewer than 8 vectors (the gather mat-vec with the gate rows riding along, matrices with
// long rows): 8 / NV warps share a vector, each a column part, and only the warps working on ONE output row (its up and gate
// vectors, all parts) meet, at a named barrier of their own, before one of them combines the sums; the stage goes back
// through the "empty" mbarrier as above.
template <int WT, bool SPARSE, bool GATED>
__global__ void __launch_bounds__(RING_THREADS) k_gemv_ring_g(const RingP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float s_grp[2][RING_WARPS][RING_WARPS];              // [stage parity][vector][column part]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages, R = p.R;
    constexpr int NM = GATED ? 2 : 1;
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    uint64_t * empty = reinterpret_cast<uint64_t *>(smem + 128);
    int * items = reinterpret_cast<int *>(smem + 8 * 32);
    const size_t x_bytes = WT == PI_TYPE_F16 ? (size_t)p.ncols * 2 : (size_t)p.nb * 40;
    unsigned char * xs = smem + (((size_t)8 * 32 + (size_t)4 * p.max_items + 127) & ~(size_t)127);
    unsigned char * ring = xs + ((x_bytes + 127) & ~(size_t)127);

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) { mbar_init(full + s, 1); mbar_init(empty + s, RING_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    int n_items, n_stages;
    auto stage_first = [&](int st) { return (cta + st * G) * R; };
    auto issue = [&](int st) {                                       // all lanes of warp 0
        const int s = st % S, first = stage_first(st), n = min(R, n_items - first);
        unsigned char * dstp = ring + (size_t)s * p.stage_bytes;
        if (!SPARSE) {
            if (lane == 0) {
                mbar_expect_tx(full + s, (unsigned)(n * p.row_bytes));
                bulk_g2s(dstp, p.W + (size_t)first * p.row_bytes, (unsigned)(n * p.row_bytes), full + s);
            }
        } else {
            if (lane == 0) mbar_expect_tx(full + s, (unsigned)(n * NM * p.row_bytes));
            for (int k = lane; k < n; k += 32) {
                const int r = items[st * R + k];
                bulk_g2s(dstp + (size_t)k * p.row_bytes, p.W + (size_t)r * p.row_bytes, (unsigned)p.row_bytes, full + s);
                if (GATED) bulk_g2s(dstp + (size_t)(R + k) * p.row_bytes, p.W2 + (size_t)r * p.row_bytes, (unsigned)p.row_bytes, full + s);
            }
        }
    };
    if (!SPARSE) {
        n_items = p.nrows;
        const int total_stages = (n_items + R - 1) / R;
        n_stages = cta < total_stages ? (total_stages - cta + G - 1) / G : 0;
        const int pre = p.pre < 0 ? S : min(p.pre, S);
        if (warp == 0) for (int st = 0; st < pre && st < n_stages; st++) issue(st);
    }
    pdl_wait();
    if (!SPARSE && p.pre >= 0 && warp == 0) for (int st = min(p.pre, S); st < S && st < n_stages; st++) issue(st);
    if (SPARSE) {
        // the list entry this thread would own is read together with the count, not after it (the list buffer has nrows
        // entries whatever the count; entries beyond the count are stale and dropped below): one round trip, not two
        int spec = 0;
        {
            const int it = stage_first(tid / R) + (tid % R);
            if (tid < p.max_items && it < p.nrows) spec = p.list[it];
        }
        n_items = min(*p.count, p.nrows);
        const int total_stages = (n_items + R - 1) / R;
        n_stages = cta < total_stages ? (total_stages - cta + G - 1) / G : 0;
        n_stages = min(n_stages, p.max_items / R);
        for (int i = tid; i < n_stages * R; i += RING_THREADS) {
            const int it = stage_first(i / R) + (i % R);
            int r = it < n_items ? (i == tid ? spec : p.list[it]) : 0;
            items[i] = (unsigned)r < (unsigned)p.nrows ? r : 0;
        }
        __syncthreads();
        if (warp == 0) for (int st = 0; st < S && st < n_stages; st++) issue(st);
    }
    if (WT == PI_TYPE_F16) {
        const uint4 * src = reinterpret_cast<const uint4 *>(p.x.h16);
        uint4 * dstx = reinterpret_cast<uint4 *>(xs);
        for (int i = tid; i < p.ncols / 8; i += RING_THREADS) dstx[i] = src[i];
    } else {
        uint4 * lo = reinterpret_cast<uint4 *>(xs);
        uint4 * hi = lo + p.nb;
        uint2 * ds = reinterpret_cast<uint2 *>(hi + p.nb);
        for (int i = tid; i < p.nb; i += RING_THREADS) {
            lo[i] = p.x.lo[i]; hi[i] = p.x.hi[i];
            ds[i] = make_uint2(__float_as_uint(p.x.d[i]), (unsigned)p.x.s[i]);
        }
    }
    __syncthreads();

    const int units = WT == PI_TYPE_F16 ? p.ncols / 8 : p.nb;
    const int NV = R * NM, wpv = RING_WARPS / NV;                   // warps per vector
    const int vec = warp / wpv, part = warp % wpv, k = vec % R;     // my vector of the stage, my column part, its output row
    const int per = units / wpv, gw = NM * wpv;                     // units per part, warps working on one output row
    bool dead = false;                                              // warp-uniform
    for (int st = 0; st < n_stages; st++) {
        const int s = st % S;
        const unsigned parity = (unsigned)(st / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            dead = __any_sync(0xffffffffu, gave_up) != 0;
            if (dead && lane == 0) atomicOr(p.status, 4u);
        }
        const unsigned char * base = ring + (size_t)s * p.stage_bytes;
        const int first = stage_first(st);
        const int n = min(R, n_items - first);
        float v = 0.f;
        if (!dead && k < n) {
            float acc[1];
            ring_dot_rows<WT, 1>(base + (size_t)vec * p.row_bytes, (size_t)p.row_bytes, part * per, (part + 1) * per, p.nb, xs, lane, acc);
            v = warp_sum(acc[0]);
        }
        if (gw > 1) {                                                // the warps of output row k meet; nobody else waits
            if (lane == 0) s_grp[st & 1][vec][part] = v;
            asm volatile("bar.sync %0, %1;" :: "r"(1 + k), "r"(gw * 32) : "memory");
        }
        if (vec < R && part == 0 && lane == 0 && k < n && !dead) {
            float v2 = 0.f;
            if (gw > 1) {
                v = s_grp[st & 1][k][0];
                for (int q = 1; q < wpv; q++) v += s_grp[st & 1][k][q];
                if (GATED) { v2 = s_grp[st & 1][R + k][0]; for (int q = 1; q < wpv; q++) v2 += s_grp[st & 1][R + k][q]; }
            }
            const int r = SPARSE ? items[st * R + k] : first + k;
            const int64_t g = SPARSE && p.bucket ? p.bucket[r] : r;
            float o = v;                                             // batch 1: a listed row is an active row
            if (GATED) o = fmaxf(v2, 0.f) * v;
            if (p.bias) o += p.bias[g];
            if (p.relu) o = fmaxf(o, 0.f);
            if (p.dst)   p.dst[g] = o;
            if (p.dst16) p.dst16[g] = __float2half_rn(o);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        if (warp == 0 && st + S < n_stages) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(empty + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            if (gave_up) { if (lane == 0) atomicOr(p.status, 4u); }
            else if (!dead) issue(st + S);
        }
    }
    if (__syncthreads_or(dead) && tid == 0) {
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
}

struct RingPlan { bool ok; int R, split, rw, stages, ctas_per_sm; size_t stage_bytes, smem; int max_items; };

template <int WT, bool SPARSE, bool GATED>
static int launch_ring_g(const RingP & p, const RingPlan & pl, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_gemv_ring_g<WT, SPARSE, GATED>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(sm_count() * pl.ctas_per_sm), dim3(RING_THREADS), pl.smem, st, pdl, p));
    return PI_OK;
}


// Two 100 KB rings per SM rather than one big one (PI_RING_CPS / PI_RING_KB override): with a single 8-warp CTA the
// consumers are issue-latency bound, and what matters for bandwidth is ~200 KB of copies in flight per SM; four 54 KB rings
// measure the same, two 54 KB rings 30 % slower.
static RingPlan ring_plan(int wtype, int64_t nrows, int64_t ncols, bool sparse, bool gated) {
    RingPlan pl{};
    const size_t row_bytes = pi_row_bytes(wtype, ncols);
    if (row_bytes % 16 != 0) return pl;
    const int units = wtype == PI_TYPE_F16 ? (int)(ncols / 8) : (int)(ncols / QK);
    const int nm = gated ? 2 : 1;
    const size_t x_bytes = wtype == PI_TYPE_F16 ? (size_t)ncols * 2 : (size_t)(ncols / QK) * 40;
    static int cps0 = 0, kb0 = 0, rw0 = 2;
    if (!cps0) { const char * w = getenv("PI_RING_RW"); rw0 = w ? atoi(w) : 2; if (rw0 != 1 && rw0 != 4) rw0 = 2; }
    if (!cps0) { const char * v = getenv("PI_RING_CPS"); cps0 = v ? atoi(v) : 2; const char * k = getenv("PI_RING_KB"); kb0 = k ? atoi(k) : 100; }
    for (int cps = cps0; cps >= 1; cps /= 2) {
        const size_t budget = (size_t)(cps == cps0 ? kb0 : (cps == 2 ? 110 : 200)) * 1024;
        const int G = sm_count() * cps;
        int R = 1;
        while (R < 64 && (size_t)(2 * R) * nm * row_bytes <= (budget <= 64 * 1024 ? 19 : 36) * 1024) R *= 2;
        // a small dense matrix (a rank's share in a sharded run): rather more, smaller stages than CTAs without any
        static int small_on = -1;                                    // PI_RING_SMALL=0: keep the large stages (diagnostic)
        if (small_on < 0) { const char * v = getenv("PI_RING_SMALL"); small_on = !(v && v[0] == '0'); }
        while (small_on && !sparse && R > RING_WARPS && (nrows + R - 1) / R < G) R /= 2;
        // RW vectors per warp (register blocking), `split` warps per group of RW; a warp's column share stays >= 32 units
        const int nv = R * nm;
        if (nv > RING_MAX_VEC) continue;
        int rw = nv < rw0 ? nv : rw0, split = 1;
        for (;; rw /= 2) {
            const int groups = nv / rw;
            split = groups >= RING_WARPS ? 1 : RING_WARPS / groups;
            if ((units % split == 0 && units / split >= 32) || rw == 1) break;
        }
        if (units % split != 0) continue;
        const int max_items = sparse ? (int)((((nrows + G - 1) / G + R - 1) / R + 1) * R) : 0;
        if (max_items > RING_MAX_ITEMS) continue;
        const size_t head = (((size_t)8 * 32 + (size_t)4 * max_items + 127) & ~size_t(127)) + ((x_bytes + 127) & ~size_t(127));
        const size_t stage_bytes = ((size_t)R * nm * row_bytes + 127) & ~size_t(127);
        if (head + 2 * stage_bytes > budget) continue;
        int S = (int)((budget - head) / stage_bytes);
        pl.stages = S > 8 ? 8 : S;
        pl.R = R; pl.split = split; pl.rw = rw; pl.ctas_per_sm = cps; pl.max_items = max_items; pl.stage_bytes = stage_bytes;
        pl.smem = head + (size_t)pl.stages * stage_bytes;
        pl.ok = true;
        return pl;
    }
    return pl;
}

template <int WT, bool SPARSE, bool GATED, int RW>
static int launch_ring_inst(const RingP & p, const RingPlan & pl, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_gemv_ring<WT, SPARSE, GATED, RW>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() * pl.ctas_per_sm); cfg.blockDim = dim3(RING_THREADS); cfg.dynamicSmemBytes = pl.smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    PI_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return PI_OK;
}

// PI_ERR_UNSUPPORTED: shape not eligible, the caller uses the register-streaming kernel instead
int launch_gemv_ring(const GemvArgs & a, unsigned int * status, bool pdl, cudaStream_t st, bool * wrote_masks) {
    if (wrote_masks) *wrote_masks = false;
    if (a.T != 1 || !status) return PI_ERR_UNSUPPORTED;
    const bool sparse = a.list != nullptr, gated = a.W2 != nullptr;
    const RingPlan pl = ring_plan(a.wtype, a.nrows, a.ncols, sparse, gated);
    if (!pl.ok) return PI_ERR_UNSUPPORTED;
    RingP p;
    p.W = (const uint8_t *)a.W; p.W2 = (const uint8_t *)a.W2; p.row_bytes = (int64_t)pi_row_bytes(a.wtype, a.ncols);
    p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.nb = (int)(a.ncols / QK); p.x = a.x;
    p.list = a.list; p.count = a.count; p.bucket = a.bucket; p.idx = a.idx; p.threshold = a.threshold;
    p.bias = a.bias; p.relu = a.relu; p.dst = a.dst; p.dst16 = a.dst16; p.status = status;
    p.masks_out = nullptr; p.masks_threshold = a.masks_threshold;
    p.pre = a.pre_stages;
    p.R = pl.R; p.split = pl.split; p.stages = pl.stages; p.max_items = pl.max_items; p.stage_bytes = pl.stage_bytes;
    const bool q4 = a.wtype == PI_TYPE_Q4_0;
    {
        static int warp_rows = -1;
        if (warp_rows < 0) { const char * v = getenv("PI_RING_W"); warp_rows = !(v && v[0] == '0'); }
        if (warp_rows && !sparse && pl.R >= RING_WARPS && pl.stages <= 8) {
            static bool attr_w[2][16] = {{false}};
            int dev = 0;
            PI_CUDA(cudaGetDevice(&dev));
            if (dev >= 0 && dev < 16 && !attr_w[q4][dev]) {
                if (q4) PI_CUDA(cudaFuncSetAttribute(k_gemv_ring_w<PI_TYPE_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
                else    PI_CUDA(cudaFuncSetAttribute(k_gemv_ring_w<PI_TYPE_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
                attr_w[q4][dev] = true;
            }
            const dim3 grid(sm_count() * pl.ctas_per_sm);
            if (pl.R == 8 || pl.R == 16 || pl.R == 32 || pl.R == 64) {      // a stage's rows are whole bytes of the masks
                p.masks_out = a.masks_out;
                if (wrote_masks) *wrote_masks = a.masks_out != nullptr;
            }
            if (q4) PI_CUDA(launch_k(k_gemv_ring_w<PI_TYPE_Q4_0>, grid, dim3(RING_THREADS), pl.smem, st, pdl, p));
            else    PI_CUDA(launch_k(k_gemv_ring_w<PI_TYPE_F16>, grid, dim3(RING_THREADS), pl.smem, st, pdl, p));
            return PI_OK;
        }
    }
    {
        static int grp = -1;
        if (grp < 0) { const char * v = getenv("PI_RING_G"); grp = !(v && v[0] == '0'); }
        const int nv = pl.R * (gated ? 2 : 1);
        const int units = q4 ? (int)(a.ncols / QK) : (int)(a.ncols / 8);
        if (grp && pl.stages <= 8 && nv <= RING_WARPS && RING_WARPS % nv == 0 &&
            units % (RING_WARPS / nv) == 0 && (sparse || pl.R < RING_WARPS)) {
            if (!sparse) return q4 ? launch_ring_g<PI_TYPE_Q4_0, false, false>(p, pl, pdl, st) : launch_ring_g<PI_TYPE_F16, false, false>(p, pl, pdl, st);
            if (gated)   return q4 ? launch_ring_g<PI_TYPE_Q4_0, true, true>(p, pl, pdl, st) : launch_ring_g<PI_TYPE_F16, true, true>(p, pl, pdl, st);
            return q4 ? launch_ring_g<PI_TYPE_Q4_0, true, false>(p, pl, pdl, st) : launch_ring_g<PI_TYPE_F16, true, false>(p, pl, pdl, st);
        }
    }
#define PI_RING_DISPATCH_RW(RW)                                                                                                            \
    do {                                                                                                                                   \
        if (!sparse) return q4 ? launch_ring_inst<PI_TYPE_Q4_0, false, false, RW>(p, pl, pdl, st)                                          \
                               : launch_ring_inst<PI_TYPE_F16, false, false, RW>(p, pl, pdl, st);                                          \
        if (gated)   return q4 ? launch_ring_inst<PI_TYPE_Q4_0, true, true, RW>(p, pl, pdl, st)                                            \
                               : launch_ring_inst<PI_TYPE_F16, true, true, RW>(p, pl, pdl, st);                                            \
        return q4 ? launch_ring_inst<PI_TYPE_Q4_0, true, false, RW>(p, pl, pdl, st)                                                        \
                  : launch_ring_inst<PI_TYPE_F16, true, false, RW>(p, pl, pdl, st);                                                        \
    } while (0)
    if (pl.rw == 4) PI_RING_DISPATCH_RW(4);
    if (pl.rw == 2) PI_RING_DISPATCH_RW(2);
    PI_RING_DISPATCH_RW(1);
#undef PI_RING_DISPATCH_RW
}

}  // namespace pi
