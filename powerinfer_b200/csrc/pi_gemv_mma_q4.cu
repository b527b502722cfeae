// Q4_0 small-batch mat-mat (2..8 tokens per launch) with the integer dots on the tensor cores.
//
// The CPU path multiplies a Q4_0 row with a Q8_0 activation block by block: an exact integer dot of 32 nibbles with 32
// int8 values, minus 8 x (sum of the int8 values), times the two block scales, accumulated in FP32 (ggml.c:2494-2560).
// On the CUDA cores every (row, block, token) costs eight dp4a plus two 128-bit shared-memory reads of the activation
// block; at 8 tokens that kernel is bound by shared-memory bandwidth at about an eighth of the HBM rate.  Here one
// mma.sync.m16n8k32 (u8 x s8 -> s32) does the 32-value dots of 16 weight rows with 8 tokens at once: the nibbles are the
// A operand (low nibbles = values 0..15 of the block, high nibbles = values 16..31, which is exactly the k order of the
// fragment), the two int8 planes of the activations the B operand.  The integer results are the same numbers dp4a gives;
// the scales are applied per block in FP32 as before, so only the order of the FP32 additions over the blocks differs.
//
// Work unit: a tile of 16 row vectors (dense / ggml_mul_mat_idx: 16 rows; with a gate matrix: 8 up rows + the 8 gate rows
// of the same neurons), each whole row placed by one cp.async.bulk (plain, non-tensor, no multicast; 16-byte aligned) at a
// pitch that keeps the fragment reads bank-conflict free; two such stages (74 KB each at 8192 columns) fit next to the
// activation planes of the launch's tokens, which are staged once per CTA, interleaved by token.  Rows too long for that
// go in tiles of 8 vectors (rows 8..15 of the mma tile then stay zero).  16 compute warps split the blocks of a row; a
// 17th warp issues the copies, adds the partial sums in warp order through shared memory and runs the epilogue
// (predicate, gate, bias, relu) while the compute warps go on with the next tile.  Tiles are dealt round-robin to one CTA
// per SM.  Dense weights do not depend on the previous kernel: their copies are issued before griddepcontrol.wait.
// Every mbarrier wait is bounded: on expiry the warp sets bit 3 of *status and contributes zeros.
#include "pi_common.cuh"

#include <cstdlib>

namespace pi {

static constexpr int Q4M_CWARPS = 16;                  // compute warps (4 per scheduler: the block loop is a chain of dependent latencies)
static constexpr int Q4M_THREADS = (Q4M_CWARPS + 1) * 32;   // + the serving warp
static constexpr int QK = 32;                          // values of a Q4_0 / Q8_0 block
static constexpr int Q4M_TOK = 8;                      // tokens of one launch (the n extent of the fragment)

// D = A x B + C for a 16 x 32 u8 tile, a 32 x 8 s8 tile and s32 accumulators (fragment rows g and g+8, columns 2q, 2q+1)
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1,
                                         int k0, int k1, int k2, int k3) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(k0), "r"(k1), "r"(k2), "r"(k3));
}

// a packed {FP16 scale | 0x8000 - 8*s} word -> the mma's C operand, and the scale
__device__ __forceinline__ int q_magic(uint32_t w) { return (int)__byte_perm(w, 0x4B400000u, 0x7610); }
__device__ __forceinline__ float q_scale(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }
static constexpr float Q4M_BIAS = 12582912.0f + 32768.0f;

struct Q4mP {
    const uint8_t * W; const uint8_t * W2; Act x;                // x: planes of this launch's first token
    int64_t row_bytes; int nrows; int nb; int T;                 // T <= 8 tokens
    const int32_t * list; const int32_t * count; const int32_t * bucket;
    const float * idx; int64_t idx_stride; float threshold;
    const float * bias; int relu;
    float * dst; __half * dst16; int64_t dst_stride;
    unsigned int * status;
    int stages, pitch, max_tiles; size_t stage_bytes;
};

__device__ __forceinline__ void q_bar_sync(int id, int n)   { asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void q_bar_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" :: "r"(id), "r"(n) : "memory"); }
// arrive only once v0 and v1 exist, i.e. once the shared-memory loads they were summed from have returned
__device__ __forceinline__ void q_bar_arrive_after(int id, int n, float v0, float v1, float v2, float v3) {
    asm volatile("bar.arrive %0, %1;" :: "r"(id), "r"(n), "f"(v0), "f"(v1), "f"(v2), "f"(v3) : "memory");
}

// Warp roles: warps 0..15 compute (each owns every 16th pair of blocks of the tile's rows), warp 16 serves: it issues the
// copies, adds the 16 partial fragments in warp order and runs the epilogue, so the compute warps never stop at a
// block-wide barrier.  Hand-offs per tile: the compute warps write their partial sums to `red` and arrive at named
// barrier 1, where the serving warp waits; it then refills the tile's ring stage (all compute warps are past it), reads
// `red`, arrives at named barrier 2, which the compute warps pass before they write `red` for the next tile (the serving
// warp is long there by then), and stores.  All warps run the same number of tiles, so every barrier completes; a warp
// whose bounded wait for the copies ran out contributes zeros and sets bit 3 of *status.
// M16: tiles of 16 row vectors (all rows of the mma tile carry data) instead of 8; GATED: a second matrix shares the rows
// (tile = NV/2 up rows + the NV/2 gate rows of the same neurons).
template <bool SPARSE, bool GATED, bool M16>
__global__ void __launch_bounds__(Q4M_THREADS, 1) k_gemv_mma_q4(const Q4mP p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int NV = M16 ? 16 : 8;                                 // row vectors of a tile
    constexpr int IT = GATED ? NV / 2 : NV;                          // items (rows / neurons) of a tile
    constexpr int NR = M16 ? 4 : 2;                                  // accumulators of a lane
    constexpr int RW = NR * 32;                                      // floats of one warp's partial fragment
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q4 = lane & 3;                          // fragment coordinates: row / token g, word q4
    const int G = gridDim.x, cta = blockIdx.x;
    const int S = p.stages, pitch = p.pitch, nb = p.nb;
    const bool server = warp == Q4M_CWARPS;

    // shared-memory map: [S] mbarriers | row numbers of my tiles | partial sums [16 warps][RW] |
    //                    activation planes: words {lo0,hi0,..,lo3,hi3} [nb][8 tokens] 32 B, {half d | 0x8000 - 8s} [nb][8 tokens] 4 B | ring
    uint64_t * full = reinterpret_cast<uint64_t *>(smem);
    int * rows = reinterpret_cast<int *>(smem + 8 * 32);                                   // [max_tiles * IT] (sparse only)
    float * red = reinterpret_cast<float *>(smem + (((size_t)8 * 32 + (size_t)4 * IT * (SPARSE ? p.max_tiles : 0) + 127) & ~(size_t)127));
    uint4 * xw = reinterpret_cast<uint4 *>(red + Q4M_CWARPS * RW);
    uint32_t * xds = reinterpret_cast<uint32_t *>(xw + (size_t)nb * Q4M_TOK * 2);
    unsigned char * ring = reinterpret_cast<unsigned char *>(xds + (size_t)nb * Q4M_TOK);

    pdl_launch();
    if (tid == 0) {
        for (int s = 0; s < S; s++) mbar_init(full + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // stage q of this CTA = my tile number q = global tile cta + q*G
    int n_items = SPARSE ? 0 : p.nrows, my_tiles = 0;
    auto set_items = [&](int n) {
        n_items = n;
        const int tiles = (n + IT - 1) / IT;
        my_tiles = cta < tiles ? (tiles - cta + G - 1) / G : 0;
        if (SPARSE) my_tiles = min(my_tiles, p.max_tiles);
    };
    auto tile_rows = [&](int i) { return min(IT, n_items - (cta + i * G) * IT); };         // valid items of my tile i
    auto issue = [&](int i) {                                                              // all lanes of the serving warp
        const int s = i % S, n = tile_rows(i);
        unsigned char * dstp = ring + (size_t)s * p.stage_bytes;
        if (lane == 0) mbar_expect_tx(full + s, (unsigned)(n * (GATED ? 2 : 1) * p.row_bytes));
        __syncwarp();
        for (int k = lane; k < n * (GATED ? 2 : 1); k += 32) {
            const int m = k / n, kk = k % n;                                               // matrix, item within the tile
            const int r = SPARSE ? rows[i * IT + kk] : (cta + i * G) * IT + kk;
            const uint8_t * src = (m ? p.W2 : p.W) + (size_t)r * p.row_bytes;
            bulk_g2s(dstp + (size_t)(m * IT + kk) * pitch, src, (unsigned)p.row_bytes, full + s);
        }
    };

    if (!SPARSE) {
        set_items(p.nrows);
        if (server) for (int i = 0; i < S && i < my_tiles; i++) issue(i);                  // weights first: they need no producer
    }
    pdl_wait();
    if (SPARSE) {
        set_items(min(*p.count, p.nrows));
        for (int e = tid; e < my_tiles * IT; e += Q4M_THREADS) {
            const int it = (cta + (e / IT) * G) * IT + (e % IT);
            const int r = it < n_items ? p.list[it] : 0;
            rows[e] = (unsigned)r < (unsigned)p.nrows ? r : 0;
        }
        __syncthreads();
        if (server) for (int i = 0; i < S && i < my_tiles; i++) issue(i);
    }
    if (my_tiles > 0) {
        // Activation planes, interleaved by token and by lo / hi word: thread (token g, word q4) of a fragment reads its two
        // B registers as one 8-byte word, a warp reads 256 contiguous bytes.  8 consecutive threads write the 8 tokens of a
        // block (contiguous, no bank conflicts).  Scale and sum of a block are packed into one word: the FP16 scale in the
        // high half, 0x8000 - 8*s in the low half.  0x4B400000 | low half is the C operand of the mma, so the accumulator
        // comes out as the bits of 12582912.0f + 32768 + (dot - 8*s) and one FP32 subtraction replaces the integer-to-float
        // conversion (exact: the sum stays below 2^22).  Loads of 4 elements are in flight before the first store.
        const int n_el = Q4M_TOK * nb;
        for (int e0 = tid; e0 < n_el; e0 += 4 * Q4M_THREADS) {
            uint4 lo[4], hi[4];
            float dv[4];
            int sv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int e = e0 + u * Q4M_THREADS;
                const int t = e & (Q4M_TOK - 1), b = e >> 3;
                lo[u] = make_uint4(0u, 0u, 0u, 0u); hi[u] = lo[u]; dv[u] = 0.f; sv[u] = 0;
                if (e < n_el && t < p.T) {
                    lo[u] = p.x.lo[(size_t)t * nb + b]; hi[u] = p.x.hi[(size_t)t * nb + b];
                    dv[u] = p.x.d[(size_t)t * nb + b]; sv[u] = p.x.s[(size_t)t * nb + b];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int e = e0 + u * Q4M_THREADS;
                if (e < n_el) {
                    xw[(size_t)e * 2]     = make_uint4(lo[u].x, hi[u].x, lo[u].y, hi[u].y);
                    xw[(size_t)e * 2 + 1] = make_uint4(lo[u].z, hi[u].z, lo[u].w, hi[u].w);
                    xds[e] = ((uint32_t)__half_as_ushort(__float2half_rn(dv[u])) << 16) | (uint32_t)((0x8000 - 8 * sv[u]) & 0xFFFF);
                }
            }
        }
    }
    __syncthreads();
    constexpr int NB_A = 1, NB_B = 2;                                // named barriers: partial sums ready / `red` free
    constexpr int NB_COUNT = Q4M_THREADS;
    constexpr uint32_t NIB = 0x0F0F0F0Fu;

    if (!server) {
        // ------------------------------------------------------------------------------------ compute warps
        const uint2 * xb = reinterpret_cast<const uint2 *>(xw) + g * 4 + q4;              // + b*32: token g, {lo, hi} word q4
        const uint2 * xds_q = reinterpret_cast<const uint2 *>(xds) + q4;                   // + b*4: tokens 2*q4, 2*q4+1
        const int n_pairs = nb >> 1;
        for (int i = 0; i < my_tiles; i++) {
            const int s = i % S;
            bool dead = false;                                       // warp-uniform
            {
                int spins = 0;
                bool gave_up = false;
                while (!mbar_try_wait(full + s, (unsigned)(i / S) & 1u)) { if (++spins > (1 << 20)) { gave_up = true; break; } }
                dead = __any_sync(0xffffffffu, gave_up) != 0;
                if (dead && lane == 0) atomicOr(p.status, 8u);
            }
            float acc[NR];                                           // vectors g (and g+8) x tokens 2*q4, 2*q4+1
#pragma unroll
            for (int j = 0; j < NR; j++) acc[j] = 0.f;
            if (!dead) {
                const unsigned char * vrow = ring + (size_t)s * p.stage_bytes + (size_t)g * pitch;
                const uint32_t * aw = reinterpret_cast<const uint32_t *>(vrow) + q4;        // + b*4: word q4 of block b
                const __half2 * dw = reinterpret_cast<const __half2 *>(vrow + (size_t)nb * 16);   // + b/2: scales of blocks b, b+1
                const uint32_t * aw8 = reinterpret_cast<const uint32_t *>(vrow + (size_t)8 * pitch) + q4;          // vector g+8
                const __half2 * dw8 = reinterpret_cast<const __half2 *>(vrow + (size_t)8 * pitch + (size_t)nb * 16);
#pragma unroll 2
                for (int pj = warp; pj < n_pairs; pj += Q4M_CWARPS) {
                    const int b = pj * 2;
                    const uint32_t w0 = aw[b * 4], w1 = aw[b * 4 + 4];
                    const uint2 x0 = xb[b * 32], x1 = xb[b * 32 + 32];
                    const uint2 ds0 = xds_q[b * 4], ds1 = xds_q[b * 4 + 4];
                    const float2 d4 = __half22float2(dw[pj]);
                    const int k00 = q_magic(ds0.x), k01 = q_magic(ds0.y), k10 = q_magic(ds1.x), k11 = q_magic(ds1.y);
                    const float s00 = q_scale(ds0.x), s01 = q_scale(ds0.y), s10 = q_scale(ds1.x), s11 = q_scale(ds1.y);
                    int c[4], e[4];
                    if (M16) {
                        const uint32_t v0 = aw8[b * 4], v1 = aw8[b * 4 + 4];
                        const float2 e4 = __half22float2(dw8[pj]);
                        mma_u8s8(c, w0 & NIB, v0 & NIB, (w0 >> 4) & NIB, (v0 >> 4) & NIB, x0.x, x0.y, k00, k01, k00, k01);
                        mma_u8s8(e, w1 & NIB, v1 & NIB, (w1 >> 4) & NIB, (v1 >> 4) & NIB, x1.x, x1.y, k10, k11, k10, k11);
                        acc[NR - 2] = fmaf(__int_as_float(c[2]) - Q4M_BIAS, e4.x * s00, acc[NR - 2]);
                        acc[NR - 1] = fmaf(__int_as_float(c[3]) - Q4M_BIAS, e4.x * s01, acc[NR - 1]);
                        acc[NR - 2] = fmaf(__int_as_float(e[2]) - Q4M_BIAS, e4.y * s10, acc[NR - 2]);
                        acc[NR - 1] = fmaf(__int_as_float(e[3]) - Q4M_BIAS, e4.y * s11, acc[NR - 1]);
                    } else {
                        mma_u8s8(c, w0 & NIB, 0u, (w0 >> 4) & NIB, 0u, x0.x, x0.y, k00, k01, 0, 0);
                        mma_u8s8(e, w1 & NIB, 0u, (w1 >> 4) & NIB, 0u, x1.x, x1.y, k10, k11, 0, 0);
                    }
                    acc[0] = fmaf(__int_as_float(c[0]) - Q4M_BIAS, d4.x * s00, acc[0]);
                    acc[1] = fmaf(__int_as_float(c[1]) - Q4M_BIAS, d4.x * s01, acc[1]);
                    acc[0] = fmaf(__int_as_float(e[0]) - Q4M_BIAS, d4.y * s10, acc[0]);
                    acc[1] = fmaf(__int_as_float(e[1]) - Q4M_BIAS, d4.y * s11, acc[1]);
                }
            }
            if (i >= 1) q_bar_sync(NB_B, NB_COUNT);                  // the serving warp has read `red` of tile i-1
            float * r = red + (size_t)warp * RW;
#pragma unroll
            for (int j = 0; j < NR; j++) r[j * 32 + lane] = acc[j];
            __threadfence_block();
            q_bar_arrive(NB_A, NB_COUNT);
        }
    } else {
        // ------------------------------------------------------------------------------------ serving warp
        // What a lane's fragment rows are: M16 dense: items g and g+8; M16 gated: item g (up in rows g, gate in rows g+8);
        // 8 vectors dense: item g; 8 vectors gated: item g & 3 (up in lanes with g < 4, its gate sums 16 lanes up).
        constexpr int NH = (M16 && !GATED) ? 2 : 1;
        for (int i = 0; i < my_tiles; i++) {
            const int n = tile_rows(i);
            // the epilogue's global operands (row -> neuron id -> logits, bias) are fetched while the tile is computed
            const int t0 = 2 * q4, t1 = t0 + 1;
            int64_t gid[NH];
            bool mine[NH], act0[NH], act1[NH];
            float biasv[NH];
#pragma unroll
            for (int h = 0; h < NH; h++) {
                const int k = M16 ? g + 8 * h : (GATED ? (g & 3) : g);
                mine[h] = k < n && (M16 || !GATED || g < 4);
                gid[h] = 0; act0[h] = true; act1[h] = true; biasv[h] = 0.f;
                if (mine[h]) {
                    const int r = SPARSE ? rows[i * IT + k] : (cta + i * G) * IT + k;
                    gid[h] = SPARSE && p.bucket ? p.bucket[r] : r;
                    if (SPARSE) {
                        if (t0 < p.T) act0[h] = !(p.idx[(size_t)t0 * p.idx_stride + gid[h]] < p.threshold);
                        if (t1 < p.T) act1[h] = !(p.idx[(size_t)t1 * p.idx_stride + gid[h]] < p.threshold);
                    }
                    if (p.bias) biasv[h] = p.bias[gid[h]];
                }
            }
            q_bar_sync(NB_A, NB_COUNT);                              // all compute warps are past tile i: its stage is free
            if (i + S < my_tiles) issue(i + S);
            float v[NR];
#pragma unroll
            for (int j = 0; j < NR; j++) v[j] = red[j * 32 + lane];
#pragma unroll
            for (int w = 1; w < Q4M_CWARPS; w++)
#pragma unroll
                for (int j = 0; j < NR; j++) v[j] += red[w * RW + j * 32 + lane];
            if (i + 1 < my_tiles) q_bar_arrive_after(NB_B, NB_COUNT, v[0], v[1], v[NR - 2], v[NR - 1]);
#pragma unroll
            for (int h = 0; h < NH; h++) {
                float o0 = v[2 * h], o1 = v[2 * h + 1];
                if (GATED) {
                    const float g0 = M16 ? v[NR - 2] : __shfl_down_sync(0xffffffffu, v[0], 16);
                    const float g1 = M16 ? v[NR - 1] : __shfl_down_sync(0xffffffffu, v[1], 16);
                    o0 = fmaxf(g0, 0.f) * v[0]; o1 = fmaxf(g1, 0.f) * v[1];
                }
                if (mine[h]) {
                    o0 = (act0[h] ? o0 : 0.f) + biasv[h]; o1 = (act1[h] ? o1 : 0.f) + biasv[h];
                    if (p.relu) { o0 = fmaxf(o0, 0.f); o1 = fmaxf(o1, 0.f); }
                    if (t0 < p.T) {
                        if (p.dst)   p.dst[(size_t)t0 * p.dst_stride + gid[h]] = o0;
                        if (p.dst16) p.dst16[(size_t)t0 * p.dst_stride + gid[h]] = __float2half_rn(o0);
                    }
                    if (t1 < p.T) {
                        if (p.dst)   p.dst[(size_t)t1 * p.dst_stride + gid[h]] = o1;
                        if (p.dst16) p.dst16[(size_t)t1 * p.dst_stride + gid[h]] = __float2half_rn(o1);
                    }
                }
            }
        }
    }
    __syncthreads();
    if (tid == 0 && (*(volatile unsigned int *)p.status & 8u)) {     // do not exit with copies still landing in shared memory
        for (int s = 0; s < S; s++) { int spins = 0; while (!mbar_try_wait(full + s, 0) && !mbar_try_wait(full + s, 1) && ++spins < (1 << 16)) {} }
    }
}

struct Q4mPlan { bool ok; bool m16; int stages, pitch, max_tiles; size_t stage_bytes, smem; };

static constexpr size_t Q4M_SMEM_MAX = 232448;          // 227 KB: the most dynamic shared memory a CTA can opt into

static Q4mPlan q4m_plan(int64_t nrows, int nb, bool sparse, bool gated, bool m16) {
    Q4mPlan pl{};
    if (nb <= 0 || nb % 8 != 0) return pl;                           // rows must be copyable in 16-byte units
    const int nv = m16 ? 16 : 8;
    const int it = gated ? nv / 2 : nv;
    const int G = sm_count();
    if (!sparse && nrows / it < G) return pl;                        // too few row tiles to fill the GPU
    const int max_tiles = sparse ? (int)(((nrows + it - 1) / it + G - 1) / G) : 0;
    if (max_tiles > 2048) return pl;
    const size_t row_bytes = (size_t)nb * 18;
    // pitch: the 8 vectors x 4 words of a fragment read must fall into 32 different banks
    int pitch = 0;
    for (int pad = 16; pad <= 144 && !pitch; pad += 16) {
        const int wp = (int)((row_bytes + pad) / 4);
        unsigned seen = 0;
        for (int r = 0; r < 8; r++) for (int q = 0; q < 4; q++) seen |= 1u << ((r * wp + q) & 31);
        if (seen == 0xffffffffu) pitch = (int)row_bytes + pad;
    }
    if (!pitch) return pl;
    const size_t head = (((size_t)8 * 32 + (size_t)4 * it * max_tiles + 127) & ~size_t(127))
                      + (size_t)Q4M_CWARPS * (m16 ? 128 : 64) * 4 + (size_t)nb * Q4M_TOK * 36;
    const size_t stage_bytes = ((size_t)nv * pitch + 127) & ~size_t(127);
    if (head + 2 * stage_bytes > Q4M_SMEM_MAX) return pl;
    int S = (int)((Q4M_SMEM_MAX - head) / stage_bytes);
    static int s_env = -1;
    if (s_env < 0) { const char * v = getenv("PI_MMA_Q4_STAGES"); s_env = v ? atoi(v) : 0; }
    if (s_env >= 2 && s_env < S) S = s_env;
    pl.ok = true; pl.m16 = m16; pl.stages = S > 8 ? 8 : S; pl.pitch = pitch; pl.max_tiles = max_tiles;
    pl.stage_bytes = stage_bytes; pl.smem = head + (size_t)pl.stages * stage_bytes;
    return pl;
}

template <bool SPARSE, bool GATED, bool M16>
static int launch_q4m_inst(const Q4mP & p, const Q4mPlan & pl, bool pdl, cudaStream_t st) {
    static bool attr_done[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    auto kern = k_gemv_mma_q4<SPARSE, GATED, M16>;
    if (dev >= 0 && dev < 16 && !attr_done[dev]) {
        PI_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Q4M_SMEM_MAX));
        attr_done[dev] = true;
    }
    PI_CUDA(launch_k(kern, dim3(sm_count()), dim3(Q4M_THREADS), pl.smem, st, pdl, p));
    return PI_OK;
}

template <bool M16>
static int launch_q4m_shape(const Q4mP & p, const Q4mPlan & pl, bool sparse, bool gated, bool pdl, cudaStream_t st) {
    if (!sparse) return launch_q4m_inst<false, false, M16>(p, pl, pdl, st);
    if (gated)   return launch_q4m_inst<true, true, M16>(p, pl, pdl, st);
    return launch_q4m_inst<true, false, M16>(p, pl, pdl, st);
}

// PI_ERR_UNSUPPORTED: shape not eligible, the caller uses another kernel.  Tokens go in launches of at most 8.
int launch_gemv_mma_q4(const GemvArgs & a, cudaStream_t st) {
    static int enabled = -1;
    static int min_T = 0, rows_env = 0;
    if (enabled < 0) {
        const char * m = getenv("PI_MMA_Q4_MIN_T"); if (m) min_T = atoi(m);
        const char * r = getenv("PI_MMA_Q4_ROWS"); if (r) rows_env = atoi(r);
        const char * v = getenv("PI_MMA_Q4"); enabled = !(v && v[0] == '0');
    }
    const bool sparse = a.list != nullptr, gated = a.W2 != nullptr;
    if (!enabled || a.wtype != PI_TYPE_Q4_0 || !a.status || !a.x.lo) return PI_ERR_UNSUPPORTED;
    if (a.ncols % QK != 0) return PI_ERR_UNSUPPORTED;
    const int nb = (int)(a.ncols / QK);
    // tiles of 16 vectors when their ring fits next to the activation planes (rows up to 8192 columns), else of 8
    Q4mPlan pl{};
    if (rows_env != 8) pl = q4m_plan(a.nrows, nb, sparse, gated, true);
    if (!pl.ok && rows_env != 16) pl = q4m_plan(a.nrows, nb, sparse, gated, false);
    if (!pl.ok) return PI_ERR_UNSUPPORTED;
    // measured on the 70B shape: from 2 tokens on this kernel is level with or ahead of the CUDA-core one, for the gated
    // pair from 4 tokens on
    const int need_T = min_T > 0 ? min_T : (gated ? 4 : 2);
    if (a.T < need_T) return PI_ERR_UNSUPPORTED;
    for (int t0 = 0; t0 < a.T; t0 += Q4M_TOK) {
        Q4mP p;
        p.W = (const uint8_t *)a.W; p.W2 = (const uint8_t *)a.W2;
        p.x.lo = a.x.lo + (size_t)t0 * nb; p.x.hi = a.x.hi + (size_t)t0 * nb;
        p.x.d = a.x.d + (size_t)t0 * nb;   p.x.s = a.x.s + (size_t)t0 * nb;
        p.row_bytes = (int64_t)nb * 18; p.nrows = (int)a.nrows; p.nb = nb;
        p.T = a.T - t0 < Q4M_TOK ? a.T - t0 : Q4M_TOK;
        p.list = a.list; p.count = a.count; p.bucket = a.bucket;
        p.idx = a.idx ? a.idx + (size_t)t0 * a.idx_stride : nullptr; p.idx_stride = a.idx_stride; p.threshold = a.threshold;
        p.bias = a.bias; p.relu = a.relu;
        p.dst = a.dst ? a.dst + (size_t)t0 * a.dst_stride : nullptr;
        p.dst16 = a.dst16 ? a.dst16 + (size_t)t0 * a.dst_stride : nullptr;
        p.dst_stride = a.dst_stride; p.status = a.status;
        p.stages = pl.stages; p.pitch = pl.pitch; p.max_tiles = pl.max_tiles; p.stage_bytes = pl.stage_bytes;
        const int rc = pl.m16 ? launch_q4m_shape<true>(p, pl, sparse, gated, a.pdl, st) : launch_q4m_shape<false>(p, pl, sparse, gated, a.pdl, st);
        if (rc != PI_OK) return rc;
    }
    return PI_OK;
}

}  // namespace pi
