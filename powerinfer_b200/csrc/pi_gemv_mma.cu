// FP16 small-batch mat-mat (2..32 tokens) on the tensor cores, weights streamed through a shared-memory ring.
//
// Why tensor cores for a bandwidth-bound product: on the CUDA cores every token costs its own convert + FMA per weight, so
// the register-streaming kernel's time grows linearly with the batch (measured 82 us at 8 tokens, 185 us at 16 for 86-112 MB
// of active rows).  mma.sync.m16n8k16 (FP16 x FP16 -> FP32; the products of two halves are exact in FP32, as in the CPU
// path) does 256 weights x 8 tokens per warp instruction, so the batch rides along for free and the kernel goes back to
// waiting for HBM (53 us at 8 tokens).  At one token it measures the same as the CUDA-core ring kernel, which stays the
// batch-1 path (PI_MMA_MIN_T=1 routes batch 1 here too).
//
// Work unit: a tile of 16 rows (dense: consecutive rows; ggml_mul_mat_idx: 16 consecutive entries of the active list; the
// 16 gate rows ride along when a gate matrix is given).  A tile is streamed in slices of KS columns: one ring stage holds
// the 16 (32) row slices and the T activation slices, each placed by its own cp.async.bulk (plain, non-tensor, no
// multicast; 16-byte aligned) at a pitch of KS*2+16 bytes so that ldmatrix reads are bank-conflict free.  The 8 warps
// split the 16-column steps of a slice; each keeps its accumulator fragments over all slices of the tile, then the 8
// partial fragments are added in warp order through shared memory and the epilogue (predicate, gate, bias, relu) runs.
// Tiles are dealt round-robin to the CTAs.  Dense weights do not depend on the previous kernel: their copies are issued
// before griddepcontrol.wait.  Every mbarrier wait is bounded: on expiry the CTA sets bit 3 of *status and stops.
#include "pi_common.cuh"

#include <cstdlib>

namespace pi {

static constexpr int MMA_THREADS = 256;
static constexpr int MMA_WARPS = 8;
static constexpr int MMA_MAX_TILES = 256;              // list tiles one CTA may own

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

struct MmaP {
    const uint8_t * W; const uint8_t * W2; const __half * x;     // x: FP16 [T, ncols]
    int64_t row_bytes; int nrows; int ncols; int T;
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; int64_t idx_stride; float threshold;
    const float * bias; int relu;
    float * dst; __half * dst16; int64_t dst_stride;
    unsigned int * status;
    int KS, stages, pitch; size_t stage_bytes; int max_tiles;
};

// NT = token tiles of 8 (T <= 8*NT); GATED = a second matrix shares the rows
template <int NT, bool SPARSE, bool GATED>
__global__ void __launch_bounds__(MMA_THREADS) k_gemv_mma(const MmaP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NM = GATED ? 2 : 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages, KS = p.KS, pitch = p.pitch;
    const int n_slices = p.ncols / KS;

    // shared-memory map: [S] mbarriers | row numbers of my tiles | reduction buffers | ring
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    int * rows = reinterpret_cast<int *>(smem + 8 * 32);                                   // [max_tiles * 16] (sparse only)
    float * red = reinterpret_cast<float *>(smem + (((size_t)8 * 32 + (size_t)4 * 16 * (SPARSE ? p.max_tiles : 0) + 127) & ~(size_t)127));
    constexpr int FRAG = NM * NT * 128;                                                    // floats of one warp's fragments
    float * sum = red + MMA_WARPS * FRAG;                                                  // [FRAG] after the warp-order add
    unsigned char * ring = reinterpret_cast<unsigned char *>(sum + FRAG);
    ring = reinterpret_cast<unsigned char *>(((uintptr_t)ring + 127) & ~(uintptr_t)127);

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // stage q of this CTA = slice (q % n_slices) of my tile number (q / n_slices); my tile i is global tile cta + i*G
    int n_items = SPARSE ? 0 : p.nrows, my_tiles = 0, n_stages = 0;
    auto set_items = [&](int n) {
        n_items = n;
        const int tiles = (n + 15) / 16;
        my_tiles = cta < tiles ? (tiles - cta + G - 1) / G : 0;
        if (SPARSE) my_tiles = min(my_tiles, p.max_tiles);
        n_stages = my_tiles * n_slices;
    };
    auto tile_rows = [&](int i) { return min(16, n_items - (cta + i * G) * 16); };         // valid rows of my tile i
    // weight copies of stage q (all lanes of warp 0); with_x: also the activation slices and the expect_tx
    auto issue_w = [&](int q) {
        const int s = q % S, i = q / n_slices, sl = q % n_slices;
        const int n = tile_rows(i);
        unsigned char * dstp = ring + (size_t)s * p.stage_bytes;
        const size_t col_off = (size_t)sl * KS * 2;
        for (int k = lane; k < n * NM; k += 32) {
            const int m = k / n, kk = k % n;                                              // matrix, row within the tile
            const int r = SPARSE ? rows[i * 16 + kk] : (cta + i * G) * 16 + kk;
            const uint8_t * src = (m ? p.W2 : p.W) + (size_t)r * p.row_bytes + col_off;
            bulk_g2s(dstp + (size_t)(m * 16 + kk) * pitch, src, (unsigned)(KS * 2), full + s);
        }
    };
    auto issue_x = [&](int q) {
        const int s = q % S, i = q / n_slices, sl = q % n_slices;
        const int n = tile_rows(i);
        unsigned char * dstp = ring + (size_t)s * p.stage_bytes + (size_t)(NM * 16) * pitch;
        // the phase cannot complete before this arrive, whatever has landed already
        if (lane == 0) mbar_expect_tx(full + s, (unsigned)((n * NM + p.T) * KS * 2));
        for (int t = lane; t < p.T; t += 32)
            bulk_g2s(dstp + (size_t)t * pitch, p.x + (size_t)t * p.ncols + (size_t)sl * KS, (unsigned)(KS * 2), full + s);
    };

    if (!SPARSE) {
        set_items(p.nrows);
        if (warp == 0) for (int q = 0; q < S && q < n_stages; q++) issue_w(q);            // weights first: they need no producer
    }
    pdl_wait();
    if (SPARSE) {
        set_items(min(*p.count, p.nrows));
        for (int e = tid; e < my_tiles * 16; e += MMA_THREADS) {
            const int it = (cta + (e / 16) * G) * 16 + (e % 16);
            const int r = it < n_items ? p.list[it] : 0;
            rows[e] = (unsigned)r < (unsigned)p.nrows ? r : 0;
        }
        __syncthreads();
        if (warp == 0) for (int q = 0; q < S && q < n_stages; q++) issue_w(q);
    }
    if (warp == 0) for (int q = 0; q < S && q < n_stages; q++) issue_x(q);

    float acc[NM][NT][4];
#pragma unroll
    for (int m = 0; m < NM; m++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[m][nt][j] = 0.f;

    const int ksteps = KS / 16;                                     // 16-column steps per slice, dealt to the 8 warps
    // ldmatrix row addresses inside a stage (see the fragment layouts of mma.m16n8k16)
    const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_kofs = (lane >> 4) * 8;
    const int b_row = lane & 7, b_kofs = ((lane >> 3) & 1) * 8;
    bool dead = false;                                              // warp-uniform
    for (int q = 0; q < n_stages; q++) {
        const int s = q % S, sl = q % n_slices, i = q / n_slices;
        const unsigned parity = (unsigned)(q / S) & 1u;
        if (!dead) {
            int spins = 0;
            bool gave_up = false;
            while (!mbar_try_wait(full + s, parity)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
            dead = __any_sync(0xffffffffu, gave_up) != 0;
            if (dead && lane == 0) atomicOr(p.status, 8u);
        }
        const uint32_t base = smem_u32(ring + (size_t)s * p.stage_bytes);
        if (!dead) {
            for (int ks = warp; ks < ksteps; ks += MMA_WARPS) {
                uint32_t a[NM][4];
#pragma unroll
                for (int m = 0; m < NM; m++) ldmatrix_x4(a[m], base + (uint32_t)((m * 16 + a_row) * pitch + (ks * 16 + a_kofs) * 2));
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    uint32_t b[2];
                    ldmatrix_x2(b, base + (uint32_t)((NM * 16 + nt * 8 + b_row) * pitch + (ks * 16 + b_kofs) * 2));
#pragma unroll
                    for (int m = 0; m < NM; m++) mma_16816(acc[m][nt], a[m], b);
                }
            }
        }
        const bool tile_done = sl == n_slices - 1;
        if (tile_done) {
#pragma unroll
            for (int m = 0; m < NM; m++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int j = 0; j < 4; j++) { red[warp * FRAG + ((m * NT + nt) * 4 + j) * 32 + lane] = dead ? 0.f : acc[m][nt][j]; acc[m][nt][j] = 0.f; }
        }
        __syncthreads();                                             // every warp is done with stage s (and the fragments are in `red`)
        if (warp == 0 && !dead && q + S < n_stages) { issue_w(q + S); issue_x(q + S); }
        if (tile_done) {
            for (int e = tid; e < FRAG; e += MMA_THREADS) {
                float v = red[e];
#pragma unroll
                for (int w = 1; w < MMA_WARPS; w++) v += red[w * FRAG + e];
                sum[e] = v;
            }
            __syncthreads();
            const int n = tile_rows(i);
            for (int e = tid; e < 16 * p.T; e += MMA_THREADS) {
                const int mrow = e & 15, t = e >> 4;
                if (mrow >= n) continue;
                const int nt = t >> 3, col = t & 7;
                const int fl = (mrow & 7) * 4 + (col >> 1), reg = (mrow >> 3) * 2 + (col & 1);
                const float v = sum[((0 * NT + nt) * 4 + reg) * 32 + fl];
                const int r = SPARSE ? rows[i * 16 + mrow] : (cta + i * G) * 16 + mrow;
                const int64_t g = SPARSE && p.bucket ? p.bucket[r] : r;
                bool active = true;
                if (SPARSE) active = !(p.idx[(size_t)t * p.idx_stride + g] < p.threshold);
                float o = active ? v : 0.f;
                if (GATED) {
                    const float v2 = sum[((1 * NT + nt) * 4 + reg) * 32 + fl];
                    o = active ? fmaxf(v2, 0.f) * v : 0.f;
                }
                if (p.bias) o += p.bias[g];
                if (p.relu) o = fmaxf(o, 0.f);
                if (p.dst)   p.dst[(size_t)t * p.dst_stride + g] = o;
                if (p.dst16) p.dst16[(size_t)t * p.dst_stride + g] = __float2half_rn(o);
            }
            // `red` and `sum` are rewritten only after the next tile's last stage, i.e. after at least one more barrier
        }
    }
    if (__syncthreads_or(dead) && tid == 0) {                        // do not exit with copies still landing in shared memory
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
}

struct MmaPlan { bool ok; int NT, KS, stages, pitch, max_tiles, ctas_per_sm; size_t stage_bytes, smem; };

static MmaPlan mma_plan(int64_t nrows, int64_t ncols, int T, bool sparse, bool gated) {
    MmaPlan pl{};
    if (T < 1 || T > 32 || ncols % 256 != 0) return pl;
    const int nm = gated ? 2 : 1;
    const int NT = T <= 8 ? 1 : (T <= 16 ? 2 : 4);                   // instantiated: 1, 2, 4 token tiles
    // Copies much under a few KB are limited by the copy engine's per-copy cost (measured at one token: 512-byte slices
    // 72 us, 1 KB 57 us, 2 KB 38.5 us for the same 70 MB), so the slice is as wide as a ring of >= 3 stages allows with
    // one CTA per SM and 200 KB.
    static int ks_env = -1, cps_env = -1;
    if (ks_env < 0) { const char * v = getenv("PI_MMA_KS"); ks_env = v ? atoi(v) : 0; const char * c = getenv("PI_MMA_CPS"); cps_env = c ? atoi(c) : 1; if (cps_env != 2) cps_env = 1; }
    const int cps = cps_env;
    const int G = sm_count() * cps;
    const size_t budget = (cps == 1 ? 200 : 100) * 1024;
    const int max_tiles = sparse ? (int)(((nrows + 15) / 16 + G - 1) / G) : 0;
    if (max_tiles > MMA_MAX_TILES) return pl;
    const size_t frag = (size_t)nm * NT * 128 * 4;
    const size_t head = (((size_t)8 * 32 + (size_t)4 * 16 * max_tiles + 127) & ~size_t(127)) + (MMA_WARPS + 1) * frag + 128;
    for (int KS : {2048, 1024, 512, 256}) {
        if (ks_env && KS != ks_env) continue;
        if (ncols % KS != 0) continue;
        const int pitch = KS * 2 + 16;
        const size_t stage_bytes = ((size_t)(16 * nm + 8 * NT) * pitch + 127) & ~size_t(127);
        if (head + 3 * stage_bytes > budget) continue;
        const int S = (int)((budget - head) / stage_bytes);
        pl.ok = true; pl.NT = NT; pl.KS = KS; pl.stages = S > 12 ? 12 : S; pl.pitch = pitch; pl.max_tiles = max_tiles;
        pl.ctas_per_sm = cps; pl.stage_bytes = stage_bytes; pl.smem = head + (size_t)pl.stages * stage_bytes;
        return pl;
    }
    return pl;
}

template <int NT, bool SPARSE, bool GATED>
static int launch_mma_inst(const MmaP & p, const MmaPlan & pl, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_gemv_mma<NT, SPARSE, GATED>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(sm_count() * pl.ctas_per_sm), dim3(MMA_THREADS), pl.smem, st, pdl, p));
    return PI_OK;
}

// PI_ERR_UNSUPPORTED: shape not eligible, the caller uses another kernel
int launch_gemv_mma(const GemvArgs & a, cudaStream_t st) {
    static int enabled = -1;
    static int min_T = 2;
    if (enabled < 0) { const char * v = getenv("PI_MMA"); enabled = !(v && v[0] == '0'); const char * m = getenv("PI_MMA_MIN_T"); if (m) min_T = atoi(m); }
    if (!enabled || a.T < min_T || a.wtype != PI_TYPE_F16 || !a.status || !a.x.h16) return PI_ERR_UNSUPPORTED;
    const bool sparse = a.list != nullptr, gated = a.W2 != nullptr;
    if (!sparse && a.nrows / 16 < sm_count()) return PI_ERR_UNSUPPORTED;      // too few row tiles to fill the GPU (e.g. fc1)
    if (a.nrows % 16 != 0 && !sparse) return PI_ERR_UNSUPPORTED;
    const MmaPlan pl = mma_plan(a.nrows, a.ncols, a.T, sparse, gated);
    if (!pl.ok) return PI_ERR_UNSUPPORTED;
    MmaP p;
    p.W = (const uint8_t *)a.W; p.W2 = (const uint8_t *)a.W2; p.x = a.x.h16; p.row_bytes = a.ncols * 2;
    p.nrows = (int)a.nrows; p.ncols = (int)a.ncols; p.T = a.T;
    p.list = a.list; p.count = a.count; p.bucket = a.bucket; p.idx = a.idx; p.idx_stride = a.idx_stride; p.threshold = a.threshold;
    p.bias = a.bias; p.relu = a.relu; p.dst = a.dst; p.dst16 = a.dst16; p.dst_stride = a.dst_stride; p.status = a.status;
    p.KS = pl.KS; p.stages = pl.stages; p.pitch = pl.pitch; p.stage_bytes = pl.stage_bytes; p.max_tiles = pl.max_tiles;
#define PI_MMA_DISPATCH(NT)                                                                     \
    do {                                                                                        \
        if (!sparse) return launch_mma_inst<NT, false, false>(p, pl, a.pdl, st);                \
        if (gated)   return launch_mma_inst<NT, true, true>(p, pl, a.pdl, st);                  \
        return launch_mma_inst<NT, true, false>(p, pl, a.pdl, st);                              \
    } while (0)
    if (pl.NT == 1) PI_MMA_DISPATCH(1);
    if (pl.NT == 2) PI_MMA_DISPATCH(2);
    PI_MMA_DISPATCH(4);
#undef PI_MMA_DISPATCH
}

}  // namespace pi
