// ggml_axpy for FP16 rows and 2..32 tokens on the tensor cores (ggml.c:14314-14463 is the CPU path it matches).
//
// dst[t, c] = sum over listed rows r of coef[t, r] * Wt[r, c], coef = h rounded to FP16 where the token's predictor
// logit passes the threshold, else 0.  As a matrix product: C[c, t] += A[c, r] * B[r, t] with A = the staged rows read
// TRANSPOSED (ldmatrix.trans: shared memory holds rows r, the fragment wants columns c as its rows) and B = the
// coefficients; FP16 x FP16 products are exact in FP32 and the accumulation is FP32, as on the CPU.  The CUDA-core kernel
// pays a convert + FMA per weight per token (289 us for 140 MB at 16 tokens); here the tokens ride along in the n
// dimension of one mma.
//
// A CTA owns a slice of 1024 columns and a contiguous range of the union list; it streams its rows 16 at a time
// (k = 16) through a shared-memory ring, one plain cp.async.bulk per row slice (2 KB; 16-byte aligned, no multicast),
// pitch 2064 bytes so the transposed 8x8 loads are bank-conflict free.  16 warps x 64 columns: each warp keeps 4 column
// tiles x NT token tiles of accumulators for the whole range, so nothing is reduced across warps; the per-CTA results
// go to partial[row group][token][column] and the fixed-order reduction kernel adds the groups.
// Every mbarrier wait is bounded: on expiry the CTA sets bit 4 of *status and stops.
#include "pi_common.cuh"

#include <cstdlib>

namespace pi {

static constexpr int AM_THREADS = 512;
static constexpr int AM_CW = 1024;                     // columns per CTA
static constexpr int AM_PITCH = AM_CW * 2 + 16;

__device__ __forceinline__ void am_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void am_ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void am_mma(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct AxpyMmaP {
    const uint8_t * Wt; int64_t row_bytes; int nrows, ncols, T;
    const float * h; int64_t h_stride; const float * idx; int64_t idx_stride; float threshold;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    float * partial; unsigned int * status;
    int n_cs, n_rg, stages, max_rows;                  // column slices, row groups, ring stages, list rows one CTA may own
};

// NT = token tiles of 8 (T <= 8 * NT)
template <int NT>
__global__ void __launch_bounds__(AM_THREADS) k_axpy_mma(const AxpyMmaP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int TP = NT * 8;                                       // token rows of a coefficient tile
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cs = blockIdx.x % p.n_cs, rg = blockIdx.x / p.n_cs;
    const int S = p.stages;
    // shared-memory map: [S] mbarriers | list rows | coefficient tiles [tile][token][16] | ring [S][16 rows]
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    int * rows = reinterpret_cast<int *>(smem + 8 * 32);
    __half * coef = reinterpret_cast<__half *>(smem + (((size_t)8 * 32 + (size_t)4 * p.max_rows + 127) & ~(size_t)127));
    unsigned char * ring = reinterpret_cast<unsigned char *>(coef) + (((size_t)p.max_rows * TP * 2 + 127) & ~(size_t)127);
    const size_t stage_bytes = (size_t)16 * AM_PITCH;

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    pdl_wait();
    const int n = min(*p.count, p.nrows);
    const int lo = (int)((int64_t)rg * n / p.n_rg), hi = (int)((int64_t)(rg + 1) * n / p.n_rg);
    const int n_mine = min(hi - lo, p.max_rows);
    const int n_tiles = (n_mine + 15) / 16;
    for (int i = tid; i < n_tiles * 16; i += AM_THREADS) {
        // entries past the end of a last, short tile copy the range's first row: their coefficients are 0, and 0 times a
        // finite weight is 0 (stale shared memory could hold anything)
        const int r = p.list[lo + (i < n_mine ? i : 0)];
        rows[i] = (unsigned)r < (unsigned)p.nrows ? r : 0;
    }
    __syncthreads();
    auto issue = [&](int k) {                                        // all lanes of warp 0
        const int s = k % S;
        if (lane == 0) mbar_expect_tx(full + s, (unsigned)(16 * AM_CW * 2));
        if (lane < 16)
            bulk_g2s(ring + s * stage_bytes + (size_t)lane * AM_PITCH,
                        p.Wt + (size_t)rows[k * 16 + lane] * p.row_bytes + (size_t)cs * AM_CW * 2, (unsigned)(AM_CW * 2), full + s);
    };
    if (warp == 0) for (int k = 0; k < S && k < n_tiles; k++) issue(k);
    // coefficients while the first rows fly in (warp 0 joins when it is done issuing)
    for (int e = tid; e < n_tiles * 16 * TP; e += AM_THREADS) {
        const int r = e & 15, t = (e >> 4) % TP, i = (e / (16 * TP)) * 16 + r;
        float c = 0.f;
        if (i < n_mine && t < p.T) {
            const int64_t g = p.bucket ? p.bucket[rows[i]] : rows[i];
            if (!(p.idx[(size_t)t * p.idx_stride + g] < p.threshold)) c = p.h[(size_t)t * p.h_stride + g];
        }
        coef[e] = __float2half_rn(c);
    }
    __syncthreads();

    float acc[4][NT][4];
#pragma unroll
    for (int mt = 0; mt < 4; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[mt][nt][j] = 0.f;
    const int j8 = lane >> 3;
    const uint32_t a_off = (uint32_t)((((j8 >> 1) * 8 + (lane & 7)) * AM_PITCH) + (warp * 64 + (j8 & 1) * 8) * 2);
    const uint32_t b_off = (uint32_t)((((lane & 7) * 16) + ((lane >> 3) & 1) * 8) * 2);
    bool dead = false;                                               // warp-uniform
    for (int k = 0; k < n_tiles; k++) {
        const int s = k % S;
        const unsigned parity = (unsigned)(k / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            dead = __any_sync(0xffffffffu, gave_up) != 0;
            if (dead && lane == 0) atomicOr(p.status, 16u);
        }
        if (!dead) {
            const uint32_t stage = smem_u32(ring + s * stage_bytes);
            const uint32_t ct = smem_u32(coef + (size_t)k * TP * 16);
            uint32_t b[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) am_ldmatrix_x2(b[nt], ct + (uint32_t)(nt * 8 * 16 * 2) + b_off);
#pragma unroll
            for (int mt = 0; mt < 4; mt++) {
                uint32_t a[4];
                am_ldmatrix_x4_trans(a, stage + a_off + (uint32_t)(mt * 16 * 2));
#pragma unroll
                for (int nt = 0; nt < NT; nt++) am_mma(acc[mt][nt], a, b[nt]);
            }
        }
        if (k + S < n_tiles) {                                       // block-uniform: the stage is reused
            __syncthreads();
            if (warp == 0 && !dead) issue(k + S);
        }
    }
    if (__syncthreads_or(dead) && tid == 0) {                        // do not exit with copies still landing in shared memory
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
    // fragment element (row = column c of the slice, col = token): c0 (g, 2q) c1 (g, 2q+1) c2 (g+8, 2q) c3 (g+8, 2q+1)
    const int g4 = lane >> 2, q4 = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 4; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = nt * 8 + q4 * 2 + (j & 1);
                const int c = cs * AM_CW + warp * 64 + mt * 16 + g4 + (j >> 1) * 8;
                if (t < p.T) p.partial[((size_t)rg * p.T + t) * p.ncols + c] = dead ? 0.f : acc[mt][nt][j];
            }
}

// ---- Q4_0 rows.  Same product, but the staged rows are 4-bit blocks: a stage (16 rows x 1024 columns = 16 x (512 B of
// nibbles + 64 B of scales)) arrives by 16-byte cp.async from all threads (its pieces are too small for the bulk-copy
// engine: ~80 ns per copy), is expanded once into an FP16 tile w = fp16(d * (q - 8)) (one rounding: q - 8 is exact in FP16),
// and the tile is consumed exactly like the FP16 kernel's stage.  Coefficients are fp16(b8 * d8) of the CPU path's int8 x
// scale pair.  Two roundings to 11 bits that the CPU path does not have (it multiplies (q-8)*b8 as integers): relative
// error <= 5e-4 per term, far inside the Q4_0 parity bar, and only on this batched path.
static constexpr int AQ_RAW_ROW = 576;                 // bytes of a staged row slice: 32 blocks x 16 B + 32 x 2 B
static constexpr int AQ_RAW_STAGE = 16 * AQ_RAW_ROW;

struct AxpyMmaQ4P {
    const uint8_t * Wt; int64_t row_bytes; int nrows, ncols, nb, T;
    const int8_t * cq; const float * cd; int64_t c_stride; const float * idx; int64_t idx_stride; float threshold;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    float * partial;
    int n_cs, n_rg, stages, max_rows;
};

__device__ __forceinline__ void aq_cp16(void * dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory");
}

template <int NT>
__global__ void __launch_bounds__(AM_THREADS) k_axpy_mma_q4(const AxpyMmaQ4P p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int TP = NT * 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cs = blockIdx.x % p.n_cs, rg = blockIdx.x / p.n_cs;
    const int S = p.stages;
    // shared-memory map: list rows | coefficient tiles | raw ring [S][16 x 576 B] | FP16 tile [16][pitch]
    int * rows = reinterpret_cast<int *>(smem);
    __half * coef = reinterpret_cast<__half *>(smem + (((size_t)4 * p.max_rows + 127) & ~(size_t)127));
    unsigned char * raw = reinterpret_cast<unsigned char *>(coef) + (((size_t)p.max_rows * TP * 2 + 127) & ~(size_t)127);
    unsigned char * tile = raw + (size_t)S * AQ_RAW_STAGE;

    pdl_launch();
    pdl_wait();
    const int n = min(*p.count, p.nrows);
    const int lo = (int)((int64_t)rg * n / p.n_rg), hi = (int)((int64_t)(rg + 1) * n / p.n_rg);
    const int n_mine = min(hi - lo, p.max_rows);
    const int n_tiles = (n_mine + 15) / 16;
    for (int i = tid; i < n_tiles * 16; i += AM_THREADS) {
        const int r = p.list[lo + (i < n_mine ? i : 0)];             // padding entries copy a real row; their coefficient is 0
        rows[i] = (unsigned)r < (unsigned)p.nrows ? r : 0;
    }
    __syncthreads();
    auto issue = [&](int k) {                                        // all threads: 16 rows x 36 pieces of 16 bytes
        unsigned char * dst = raw + (size_t)(k % S) * AQ_RAW_STAGE;
        for (int e = tid; e < 16 * 36; e += AM_THREADS) {
            const int r = e / 36, pc = e % 36;
            const uint8_t * row = p.Wt + (size_t)rows[k * 16 + r] * p.row_bytes;
            const uint8_t * src = pc < 32 ? row + (size_t)cs * 512 + pc * 16 : row + (size_t)p.nb * 16 + (size_t)cs * 64 + (pc - 32) * 16;
            aq_cp16(dst + r * AQ_RAW_ROW + pc * 16, src);
        }
    };
    for (int k = 0; k < S - 1; k++) {
        if (k < n_tiles) issue(k);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int e = tid; e < n_tiles * 16 * TP; e += AM_THREADS) {
        const int r = e & 15, t = (e >> 4) % TP, i = (e / (16 * TP)) * 16 + r;
        float c = 0.f;
        if (i < n_mine && t < p.T) {
            const int64_t g = p.bucket ? p.bucket[rows[i]] : rows[i];
            if (!(p.idx[(size_t)t * p.idx_stride + g] < p.threshold))
                c = (float)p.cq[(size_t)t * p.c_stride + g] * p.cd[(size_t)t * (p.c_stride / 32) + g / 32];
        }
        coef[e] = __float2half_rn(c);
    }

    float acc[4][NT][4];
#pragma unroll
    for (int mt = 0; mt < 4; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[mt][nt][j] = 0.f;
    const int j8 = lane >> 3;
    const uint32_t a_off = (uint32_t)((((j8 >> 1) * 8 + (lane & 7)) * AM_PITCH) + (warp * 64 + (j8 & 1) * 8) * 2);
    const uint32_t b_off = (uint32_t)((((lane & 7) * 16) + ((lane >> 3) & 1) * 8) * 2);
    const uint32_t tile_a = smem_u32(tile);
    const __half2 off8 = __floats2half2_rn(1032.f, 1032.f);
    for (int k = 0; k < n_tiles; k++) {
        if (k + S - 1 < n_tiles) issue(k + S - 1);                   // into the slot expanded in the previous iteration
        asm volatile("cp.async.commit_group;" ::: "memory");
        // all but the S-1 most recent groups are complete: stage k has landed (for this thread's pieces)
        if (S == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else if (S == 3) asm volatile("cp.async.wait_group 2;" ::: "memory");
        else asm volatile("cp.async.wait_group 3;" ::: "memory");
        __syncthreads();                                             // everyone's pieces landed; the previous tile is consumed
        const unsigned char * rs = raw + (size_t)(k % S) * AQ_RAW_STAGE;
#pragma unroll
        for (int it = 0; it < 4; it++) {                             // 2048 outputs of 8 weights: consecutive lanes, consecutive 16 bytes
            const int e = it * AM_THREADS + tid;
            const int r = e >> 7, rem = e & 127, b = rem >> 2, pq = rem & 3;
            const uint2 w2 = *reinterpret_cast<const uint2 *>(rs + r * AQ_RAW_ROW + b * 16 + (pq & 1) * 8);
            const __half d = *reinterpret_cast<const __half *>(rs + r * AQ_RAW_ROW + 512 + b * 2);
            const __half2 d2 = __half2half2(d);
            const uint32_t sh = (pq >> 1) * 4;                       // elements 16..31 are the high nibbles
            const uint32_t x0 = w2.x >> sh, x1 = w2.y >> sh;
            auto pair = [&](uint32_t x) {                            // nibbles of bytes 0 and 1 of x -> fp16 pair d * (q - 8)
                const uint32_t bits = (x & 0x000Fu) | ((x & 0x0F00u) << 8) | 0x64006400u;      // 1024 + q, exactly
                __half2 h = *reinterpret_cast<const __half2 *>(&bits);
                h = __hmul2(__hsub2(h, off8), d2);
                return *reinterpret_cast<uint32_t *>(&h);
            };
            uint4 o;
            o.x = pair(x0); o.y = pair(x0 >> 16); o.z = pair(x1); o.w = pair(x1 >> 16);
            *reinterpret_cast<uint4 *>(tile + r * AM_PITCH + rem * 16) = o;
        }
        __syncthreads();
        const uint32_t ct = smem_u32(coef + (size_t)k * TP * 16);
        uint32_t bfr[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) am_ldmatrix_x2(bfr[nt], ct + (uint32_t)(nt * 8 * 16 * 2) + b_off);
#pragma unroll
        for (int mt = 0; mt < 4; mt++) {
            uint32_t a[4];
            am_ldmatrix_x4_trans(a, tile_a + a_off + (uint32_t)(mt * 16 * 2));
#pragma unroll
            for (int nt = 0; nt < NT; nt++) am_mma(acc[mt][nt], a, bfr[nt]);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    const int g4 = lane >> 2, q4 = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 4; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int t = nt * 8 + q4 * 2 + (j & 1);
                const int c = cs * AM_CW + warp * 64 + mt * 16 + g4 + (j >> 1) * 8;
                if (t < p.T) p.partial[((size_t)rg * p.T + t) * p.ncols + c] = acc[mt][nt][j];
            }
}

struct AxpyMmaPlan { bool ok; int NT, n_cs, n_rg, stages, max_rows; size_t smem; };

static AxpyMmaPlan axpy_mma_plan(int64_t nrows, int64_t ncols, int T, int max_groups) {
    AxpyMmaPlan pl{};
    if (T < 2 || T > 32 || ncols % AM_CW != 0) return pl;
    pl.NT = T <= 8 ? 1 : (T <= 16 ? 2 : 4);
    pl.n_cs = (int)(ncols / AM_CW);
    pl.n_rg = sm_count() / pl.n_cs;
    if (pl.n_rg < 1) pl.n_rg = 1;
    if (pl.n_rg > max_groups) pl.n_rg = max_groups;
    if (pl.n_rg < 1) return pl;
    pl.max_rows = (int)(((nrows + pl.n_rg - 1) / pl.n_rg + 1 + 15) / 16 * 16);
    const size_t head = (((size_t)8 * 32 + (size_t)4 * pl.max_rows + 127) & ~size_t(127)) + (((size_t)pl.max_rows * pl.NT * 8 * 2 + 127) & ~size_t(127));
    const size_t budget = 200 * 1024, stage = (size_t)16 * AM_PITCH;
    if (head + 2 * stage > budget) return pl;
    pl.stages = (int)((budget - head) / stage);
    if (pl.stages > 8) pl.stages = 8;
    pl.smem = head + (size_t)pl.stages * stage;
    pl.ok = true;
    return pl;
}

template <int NT>
static int launch_axpy_mma_inst(const AxpyMmaP & p, const AxpyMmaPlan & pl, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_axpy_mma<NT>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(pl.n_cs * pl.n_rg), dim3(AM_THREADS), pl.smem, st, pdl, p));
    return PI_OK;
}

template <int NT>
static int launch_axpy_mma_q4_inst(const AxpyMmaQ4P & p, int grid, size_t smem, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_axpy_mma_q4<NT>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(grid), dim3(AM_THREADS), smem, st, pdl, p));
    return PI_OK;
}

static int launch_axpy_mma_q4(const AxpyArgs & a, cudaStream_t st, int * groups_used) {
    if (!a.cq || !a.cd || a.T < 2 || a.T > 32 || a.ncols % AM_CW != 0) return PI_ERR_UNSUPPORTED;
    const int NT = a.T <= 8 ? 1 : (a.T <= 16 ? 2 : 4);
    const int n_cs = (int)(a.ncols / AM_CW);
    int n_rg = sm_count() / n_cs;
    if (n_rg > a.n_groups) n_rg = a.n_groups;
    if (n_rg < 1) return PI_ERR_UNSUPPORTED;
    const int max_rows = (int)(((a.nrows + n_rg - 1) / n_rg + 1 + 15) / 16 * 16);
    const int S = 4;
    const size_t smem = (((size_t)4 * max_rows + 127) & ~size_t(127)) + (((size_t)max_rows * NT * 8 * 2 + 127) & ~size_t(127))
                        + (size_t)S * AQ_RAW_STAGE + (size_t)16 * AM_PITCH;
    if (smem > 200 * 1024) return PI_ERR_UNSUPPORTED;
    AxpyMmaQ4P p;
    p.Wt = (const uint8_t *)a.Wt; p.row_bytes = (int64_t)pi_row_bytes(PI_TYPE_Q4_0, a.ncols); p.nrows = (int)a.nrows; p.ncols = (int)a.ncols;
    p.nb = (int)(a.ncols / 32); p.T = a.T;
    p.cq = a.cq; p.cd = a.cd; p.c_stride = a.c_stride; p.idx = a.idx; p.idx_stride = a.idx_stride; p.threshold = a.threshold;
    p.list = a.list; p.count = a.count; p.bucket = a.bucket; p.partial = a.partial;
    p.n_cs = n_cs; p.n_rg = n_rg; p.stages = S; p.max_rows = max_rows;
    if (groups_used) *groups_used = n_rg;
    if (NT == 1) return launch_axpy_mma_q4_inst<1>(p, n_cs * n_rg, smem, a.pdl, st);
    if (NT == 2) return launch_axpy_mma_q4_inst<2>(p, n_cs * n_rg, smem, a.pdl, st);
    return launch_axpy_mma_q4_inst<4>(p, n_cs * n_rg, smem, a.pdl, st);
}

// PI_ERR_UNSUPPORTED: shape not eligible, the caller uses the CUDA-core kernel
int launch_axpy_mma(const AxpyArgs & a, cudaStream_t st, int * groups_used) {
    static int enabled = -1;
    if (enabled < 0) { const char * v = getenv("PI_MMA"); enabled = !(v && v[0] == '0'); }
    if (enabled && a.wtype == PI_TYPE_Q4_0) return launch_axpy_mma_q4(a, st, groups_used);
    if (!enabled || a.wtype != PI_TYPE_F16 || !a.status || !a.h) return PI_ERR_UNSUPPORTED;
    const AxpyMmaPlan pl = axpy_mma_plan(a.nrows, a.ncols, a.T, a.n_groups);
    if (!pl.ok) return PI_ERR_UNSUPPORTED;
    AxpyMmaP p;
    p.Wt = (const uint8_t *)a.Wt; p.row_bytes = a.ncols * 2; p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.T = a.T;
    p.h = a.h; p.h_stride = a.h_stride; p.idx = a.idx; p.idx_stride = a.idx_stride; p.threshold = a.threshold;
    p.list = a.list; p.count = a.count; p.bucket = a.bucket; p.partial = a.partial; p.status = a.status;
    p.n_cs = pl.n_cs; p.n_rg = pl.n_rg; p.stages = pl.stages; p.max_rows = pl.max_rows;
    if (groups_used) *groups_used = pl.n_rg;
    if (pl.NT == 1) return launch_axpy_mma_inst<1>(p, pl, a.pdl, st);
    if (pl.NT == 2) return launch_axpy_mma_inst<2>(p, pl, a.pdl, st);
    return launch_axpy_mma_inst<4>(p, pl, a.pdl, st);
}

}  // namespace pi
