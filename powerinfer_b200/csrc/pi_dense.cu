// Dense decode nodes between the sparse operators: normalisation (with the residual / partial-sum reduction that
// precedes it fused in), RoPE, KV store and one-token attention.  All are latency-bound at batch 1; they exist to
// keep the residual stream on the device and to hand the next mat-vec its input already in FP16 / Q8_0 form.
#include "pi_common.cuh"

#include <cstdlib>

namespace pi {

static constexpr int QK = 32;

// ------------------------------------------------------------------------------------------------
// llm_build_norm (llama.cpp:4420-4450) = ggml_rms_norm | ggml_norm, * weight, + bias, with the CPU path's numerics
// (ggml.c:9169-9284): squares / deviations are formed in float, summed in double, scale = 1/sqrtf(mean + eps).
// Optional prologue: v = sum_j partial[j] (+ in_bias) (+ residual), written back as the new residual stream.
// Optional epilogue: the normalised vector as FP16 or Q8_0 planes for the mat-vec that consumes it.
// One CTA per token; a thread owns up to NORM_CHUNKS groups of 8 consecutive values.
static constexpr int NORM_CHUNKS = 2;

struct NormP {
    const float * x; int64_t n; int rms; float eps; const float * w; const float * b;
    const float * partial; int n_groups; int T; const float * residual; const float * residual2; const float * in_bias; float * x_out;
    int64_t partial_stride; unsigned int * status;
    // exchange (see NormArgs): mailboxes of every rank, this rank's own, the step counter
    int x_ranks, x_rank, x_index, x_per_step; int64_t x_slot; long long x_wait;
    unsigned int * x_mbox[PI_MAX_RANKS]; const unsigned int * x_mbox_local;
    const unsigned int * x_step; const float * x_extra;
    float * y; int act_type; ActBuf act; int act2_type; ActBuf act2; int act2_src;
};

__device__ __forceinline__ double block_sum_d(double v, double * s_red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum_d(v);
    __syncthreads();                       // s_red may still be read from a previous call
    if (lane == 0) s_red[wid] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < nw; i++) t += s_red[i];
    return t;
}

// Emit 8 consecutive values (chunk index c8 = first column / 8) of token t as activation planes.
// Must be called by every lane of a warp (it shuffles); `valid` gates the stores.  With n % 32 == 0 the 4 lanes that
// share a Q8 block are valid or invalid together.
__device__ __forceinline__ void emit_act8(int type, const ActBuf & a, int t, int64_t n, int c8, const float (&v)[8], bool valid) {
    if (type == PI_TYPE_F16) {
        if (!valid) return;
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        *reinterpret_cast<uint4 *>(a.h16 + (size_t)t * n + (size_t)c8 * 8) = *reinterpret_cast<uint4 *>(h);
    } else if (type == PI_TYPE_Q4_0) {
        // 4 consecutive threads (lanes 4k..4k+3) hold one block of 32 values
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float d  = amax / 127.0f;
        const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
        int q[8], s = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) { q[j] = __float2int_rn(v[j] * id); s += q[j]; }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        const int nb = (int)(n / QK);
        const size_t blk = (size_t)t * nb + (c8 >> 2);
        const int part = c8 & 3;                                  // which 8 of the 32
        uint2 packed;
        packed.x = (uint32_t)(q[0] & 0xFF) | ((uint32_t)(q[1] & 0xFF) << 8) | ((uint32_t)(q[2] & 0xFF) << 16) | ((uint32_t)(q[3] & 0xFF) << 24);
        packed.y = (uint32_t)(q[4] & 0xFF) | ((uint32_t)(q[5] & 0xFF) << 8) | ((uint32_t)(q[6] & 0xFF) << 16) | ((uint32_t)(q[7] & 0xFF) << 24);
        if (!valid) return;
        uint2 * plane = reinterpret_cast<uint2 *>(part < 2 ? a.lo + blk : a.hi + blk);
        plane[part & 1] = packed;
        if (part == 0) { a.d[blk] = __half2float(__float2half_rn(d)); a.s[blk] = s; }
    }
}

// MAXT = the launch bound: 512 threads cover n <= 8192 with registers to spare for the weights, 1024 cover n <= 16384
template <int MAXT>
__global__ void __launch_bounds__(MAXT) k_norm(const NormP p) {
    __shared__ double s_red[32];
    const int t = blockIdx.x;
    const int64_t n = p.n;
    pdl_launch();
    // the norm weights are read once per step, so they are cold: ask for them before the wait (hints cost no registers)
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
        if (c < n && (threadIdx.x & 3) == 0) {
            if (p.w) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.w + c));
            if (p.b) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.b + c));
            if (p.in_bias) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.in_bias + c));
        }
    }
    pdl_wait();
    const size_t tn = p.partial_stride ? (size_t)p.partial_stride : (size_t)p.T * n;
    const float * partial = p.partial;
    // ---- all loads of all chunks first (x_out may alias the inputs, so the compiler cannot move a load across a store
    //      itself): one round trip instead of one per chunk
    float v[NORM_CHUNKS][8];
    bool ok[NORM_CHUNKS];
    float4 in[NORM_CHUNKS][2][2];                                   // [chunk][x | residual][half]
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
        ok[k] = c < n;
        const size_t o = (size_t)t * n + c;
#pragma unroll
        for (int q = 0; q < 2; q++) { in[k][q][0] = z4; in[k][q][1] = z4; }
        if (ok[k]) {
            if (!p.partial) { in[k][0][0] = *reinterpret_cast<const float4 *>(p.x + o); in[k][0][1] = *reinterpret_cast<const float4 *>(p.x + o + 4); }
            if (p.residual)  { in[k][1][0] = *reinterpret_cast<const float4 *>(p.residual + o); in[k][1][1] = *reinterpret_cast<const float4 *>(p.residual + o + 4); }
        }
    }
    auto add8 = [](float (&d)[8], const float4 a, const float4 b) {
        d[0] += a.x; d[1] += a.y; d[2] += a.z; d[3] += a.w; d[4] += b.x; d[5] += b.y; d[6] += b.z; d[7] += b.w;
    };
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
        const size_t o = (size_t)t * n + c;
#pragma unroll
        for (int j = 0; j < 8; j++) v[k][j] = 0.f;
        if (ok[k]) {
            if (p.partial) {
                for (int g = 0; g < p.n_groups; g++) {
                    const float4 a = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)g * tn + o));
                    const float4 b = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)g * tn + o + 4));
                    add8(v[k], a, b);
                }
            } else {
                add8(v[k], in[k][0][0], in[k][0][1]);
            }
            // same order of additions as the graph: bias, residual, second residual (the rarer two cost their own round trip)
            if (p.in_bias) add8(v[k], *reinterpret_cast<const float4 *>(p.in_bias + c), *reinterpret_cast<const float4 *>(p.in_bias + c + 4));
            if (p.residual) add8(v[k], in[k][1][0], in[k][1][1]);
            if (p.residual2) add8(v[k], *reinterpret_cast<const float4 *>(p.residual2 + o), *reinterpret_cast<const float4 *>(p.residual2 + o + 4));
        }
    }
    // weights (made L2-resident by the hints above): issued before the stores and the reductions so that their latency hides there
    float wv[NORM_CHUNKS][8], bv[NORM_CHUNKS][8];
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
#pragma unroll
        for (int j = 0; j < 8; j++) { wv[k][j] = 1.f; bv[k][j] = 0.f; }
        if (MAXT <= 512) {
            if (ok[k] && p.w) {
                const float4 a = *reinterpret_cast<const float4 *>(p.w + c), b = *reinterpret_cast<const float4 *>(p.w + c + 4);
                wv[k][0] = a.x; wv[k][1] = a.y; wv[k][2] = a.z; wv[k][3] = a.w; wv[k][4] = b.x; wv[k][5] = b.y; wv[k][6] = b.z; wv[k][7] = b.w;
            }
            if (ok[k] && p.b) {
                const float4 a = *reinterpret_cast<const float4 *>(p.b + c), b = *reinterpret_cast<const float4 *>(p.b + c + 4);
                bv[k][0] = a.x; bv[k][1] = a.y; bv[k][2] = a.z; bv[k][3] = a.w; bv[k][4] = b.x; bv[k][5] = b.y; bv[k][6] = b.z; bv[k][7] = b.w;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
        const size_t o = (size_t)t * n + c;
        if (ok[k] && p.x_out) {
            *reinterpret_cast<float4 *>(p.x_out + o)     = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
            *reinterpret_cast<float4 *>(p.x_out + o + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
        if (p.act2_type && p.act2_src == 0) emit_act8(p.act2_type, p.act2, t, n, (int)(c / 8), v[k], ok[k]);
    }

    PI_TL_MARK(0);
    float scale, mean = 0.f;
    if (p.rms) {
        double s = 0.0;
#pragma unroll
        for (int k = 0; k < NORM_CHUNKS; k++)
#pragma unroll
            for (int j = 0; j < 8; j++) s += (double)(v[k][j] * v[k][j]);
        s = block_sum_d(s, s_red);
        const float ms = (float)(s / (double)n);
        scale = 1.0f / sqrtf(ms + p.eps);
    } else {
        double s = 0.0;
#pragma unroll
        for (int k = 0; k < NORM_CHUNKS; k++)
#pragma unroll
            for (int j = 0; j < 8; j++) s += (double)v[k][j];           // slots beyond n hold 0
        s = block_sum_d(s, s_red);
        mean = (float)(s / (double)n);
        double s2 = 0.0;
#pragma unroll
        for (int k = 0; k < NORM_CHUNKS; k++) {
            if (!ok[k]) continue;
#pragma unroll
            for (int j = 0; j < 8; j++) { v[k][j] = v[k][j] - mean; s2 += (double)(v[k][j] * v[k][j]); }
        }
        s2 = block_sum_d(s2, s_red);
        const float var = (float)(s2 / (double)n);
        scale = 1.0f / sqrtf(var + p.eps);
    }
    PI_TL_MARK(1);
#pragma unroll
    for (int k = 0; k < NORM_CHUNKS; k++) {
        const int64_t c = ((int64_t)k * blockDim.x + threadIdx.x) * 8;
        float y[8];
        if (MAXT > 512) {                                              // no registers to hold them across the reductions
            if (ok[k] && p.w) {
                const float4 a = *reinterpret_cast<const float4 *>(p.w + c), b = *reinterpret_cast<const float4 *>(p.w + c + 4);
                wv[k][0] = a.x; wv[k][1] = a.y; wv[k][2] = a.z; wv[k][3] = a.w; wv[k][4] = b.x; wv[k][5] = b.y; wv[k][6] = b.z; wv[k][7] = b.w;
            }
            if (ok[k] && p.b) {
                const float4 a = *reinterpret_cast<const float4 *>(p.b + c), b = *reinterpret_cast<const float4 *>(p.b + c + 4);
                bv[k][0] = a.x; bv[k][1] = a.y; bv[k][2] = a.z; bv[k][3] = a.w; bv[k][4] = b.x; bv[k][5] = b.y; bv[k][6] = b.z; bv[k][7] = b.w;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float r = __fmul_rn(v[k][j], scale);                       // separate roundings, as separate graph nodes give
            if (ok[k] && p.w) r = __fmul_rn(r, wv[k][j]);
            if (ok[k] && p.b) r = __fadd_rn(r, bv[k][j]);
            y[j] = r;
        }
        if (ok[k] && p.y) {
            float * o = p.y + (size_t)t * n + c;
            *reinterpret_cast<float4 *>(o)     = make_float4(y[0], y[1], y[2], y[3]);
            *reinterpret_cast<float4 *>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
        }
        if (p.act_type) emit_act8(p.act_type, p.act, t, n, (int)(c / 8), y, ok[k]);
        if (p.act2_type && p.act2_src == 1) emit_act8(p.act2_type, p.act2, t, n, (int)(c / 8), y, ok[k]);
    }
    PI_TL_MARK(2);
}

// The same norm spread over a thread-block cluster: one SM moves the ~170 KB a norm of 8192 values touches (input,
// residual, weights, new residual stream, activation planes) in ~3 us, eight SMs in a fraction of that.  CTA `rank` of the
// cluster owns a contiguous slice of n / cluster_size values (a multiple of 256: whole Q8_0 blocks, whole warps); the
// partial sums are pushed into every CTA's shared memory (distributed shared memory) and added in rank order, so the
// result does not depend on timing.  Same order of additions and roundings per element as k_norm.
__device__ __forceinline__ unsigned cluster_rank()  { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size()  { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait()   { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// store into the same shared-memory variable of CTA `rank` of this cluster
__device__ __forceinline__ void cluster_store_f64(double * local, unsigned rank, double v) {
    unsigned la = (unsigned)__cvta_generic_to_shared(local), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
    asm volatile("st.shared::cluster.f64 [%0], %1;" :: "r"(ra), "d"(v) : "memory");
}

__global__ void __launch_bounds__(256) k_norm_cluster(const NormP p) {
    __shared__ double s_red[32];
    __shared__ double s_all[2][8];                                  // [statistic][CTA of the cluster]: every CTA's partial sums, pushed by their owners
    const unsigned rank = cluster_rank(), CS = cluster_size();
    const int t = blockIdx.x / CS;
    const int64_t n = p.n;
    const int64_t c = (int64_t)rank * (n / CS) + (int64_t)threadIdx.x * 8;      // every thread owns 8 values: blockDim = n / CS / 8
    const size_t o = (size_t)t * n + c;
    pdl_launch();
    cluster_arrive();                                                // (waited for before the first store into a peer's shared memory)
    if ((threadIdx.x & 3) == 0) {
        if (p.w) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.w + c));
        if (p.b) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.b + c));
        if (p.in_bias) asm volatile("prefetch.global.L2 [%0];" :: "l"(p.in_bias + c));
    }
    pdl_wait();
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 r0 = z4, r1 = z4;
    if (p.residual) { r0 = *reinterpret_cast<const float4 *>(p.residual + o); r1 = *reinterpret_cast<const float4 *>(p.residual + o + 4); }
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto add8 = [&](const float4 a, const float4 b) {
        v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w; v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
    };
    if (p.partial) {
        const size_t tn = p.partial_stride ? (size_t)p.partial_stride : (size_t)p.T * n;
        const float * partial = p.partial;
        constexpr int GP = 24;                                         // slots in flight per pass (the one-token sparse kernels write 12-37)
        float4 a[GP], b[GP];
        for (int g0 = 0; g0 < p.n_groups; g0 += GP) {
#pragma unroll
            for (int u = 0; u < GP; u++) {
                a[u] = z4; b[u] = z4;
                if (g0 + u < p.n_groups) {
                    a[u] = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)(g0 + u) * tn + o));
                    b[u] = __ldcg(reinterpret_cast<const float4 *>(partial + (size_t)(g0 + u) * tn + o + 4));
                }
            }
#pragma unroll
            for (int u = 0; u < GP; u++) add8(a[u], b[u]);
        }
    } else {
        add8(*reinterpret_cast<const float4 *>(p.x + o), *reinterpret_cast<const float4 *>(p.x + o + 4));
    }
    PI_TL_MARK(0);
    if (p.x_ranks > 1) {
        // ---- exchange: v is this rank's share.  Every value travels as an 8-byte pair {value, number of this exchange}
        //      (two pairs per 16-byte store), written into every other rank's mailbox with plain stores.  A pair arrives
        //      whole, so the receiver needs no flag, no fence and no barrier: each thread polls the pairs of its own 8 values
        //      in its own mailbox until they carry this exchange's number (bounded), then adds the shares in rank order.
        if (p.x_extra) add8(*reinterpret_cast<const float4 *>(p.x_extra + o), *reinterpret_cast<const float4 *>(p.x_extra + o + 4));
        const unsigned int epoch = __ldcg(p.x_step) * (unsigned)p.x_per_step + (unsigned)p.x_index + 1u;
        const unsigned int par = epoch & 1u;
        const size_t own_w = (((size_t)par * p.x_ranks + p.x_rank) * (size_t)p.x_slot + o) * 2;
        for (int q = 0; q < p.x_ranks; q++) {
            if (q == p.x_rank) continue;
            unsigned int * dst = p.x_mbox[q] + own_w;
#pragma unroll
            for (int j = 0; j < 4; j++)
                asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};"
                             :: "l"(dst + 4 * j), "r"(__float_as_uint(v[2 * j])), "r"(epoch), "r"(__float_as_uint(v[2 * j + 1])) : "memory");
        }
        uint4 w[PI_MAX_RANKS][4];
        auto fetch = [&](int q) {
            const unsigned int * src = p.x_mbox_local + (((size_t)par * p.x_ranks + q) * (size_t)p.x_slot + o) * 2;
#pragma unroll
            for (int j = 0; j < 4; j++)
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(w[q][j].x), "=r"(w[q][j].y), "=r"(w[q][j].z), "=r"(w[q][j].w) : "l"(src + 4 * j) : "memory");
        };
        auto arrived = [&](int q) {
            bool ok_all = true;
#pragma unroll
            for (int j = 0; j < 4; j++) ok_all = ok_all && (int)(w[q][j].y - epoch) >= 0 && (int)(w[q][j].w - epoch) >= 0;
            return ok_all;
        };
        unsigned int pending = 0;
#pragma unroll
        for (int q = 0; q < PI_MAX_RANKS; q++) if (q < p.x_ranks && q != p.x_rank) fetch(q);
#pragma unroll
        for (int q = 0; q < PI_MAX_RANKS; q++) if (q < p.x_ranks && q != p.x_rank && !arrived(q)) pending |= 1u << q;
        if (pending) {
            const long long t0 = clock64();
            while (pending) {
#pragma unroll
                for (int q = 0; q < PI_MAX_RANKS; q++) if (pending >> q & 1u) fetch(q);
#pragma unroll
                for (int q = 0; q < PI_MAX_RANKS; q++) if ((pending >> q & 1u) && arrived(q)) pending &= ~(1u << q);
                if (pending && clock64() - t0 > p.x_wait) break;       // never forever: the step finishes, the host reads the status
            }
            if (pending) atomicOr(p.status, 1u);
        }
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int q = 0; q < PI_MAX_RANKS; q++) {
            if (q >= p.x_ranks) continue;
            if (q == p.x_rank) {
#pragma unroll
                for (int j = 0; j < 8; j++) s[j] += v[j];
            } else {
#pragma unroll
                for (int j = 0; j < 4; j++) { s[2 * j] += __uint_as_float(w[q][j].x); s[2 * j + 1] += __uint_as_float(w[q][j].z); }
            }
        }
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = s[j];
    }
    if (p.in_bias) add8(*reinterpret_cast<const float4 *>(p.in_bias + c), *reinterpret_cast<const float4 *>(p.in_bias + c + 4));
    if (p.residual) add8(r0, r1);
    if (p.residual2) add8(*reinterpret_cast<const float4 *>(p.residual2 + o), *reinterpret_cast<const float4 *>(p.residual2 + o + 4));
    float wv[8], bv[8];
#pragma unroll
    for (int j = 0; j < 8; j++) { wv[j] = 1.f; bv[j] = 0.f; }
    if (p.w) {
        const float4 a = *reinterpret_cast<const float4 *>(p.w + c), b = *reinterpret_cast<const float4 *>(p.w + c + 4);
        wv[0] = a.x; wv[1] = a.y; wv[2] = a.z; wv[3] = a.w; wv[4] = b.x; wv[5] = b.y; wv[6] = b.z; wv[7] = b.w;
    }
    if (p.b) {
        const float4 a = *reinterpret_cast<const float4 *>(p.b + c), b = *reinterpret_cast<const float4 *>(p.b + c + 4);
        bv[0] = a.x; bv[1] = a.y; bv[2] = a.z; bv[3] = a.w; bv[4] = b.x; bv[5] = b.y; bv[6] = b.z; bv[7] = b.w;
    }
    if (p.x_out) {
        *reinterpret_cast<float4 *>(p.x_out + o)     = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p.x_out + o + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (p.act2_type && p.act2_src == 0) emit_act8(p.act2_type, p.act2, t, n, (int)(c / 8), v, true);
    PI_TL_MARK(1);

    // Every CTA gets the sum over the cluster, ranks in order.  The partial sums are PUSHED: CTA r writes its sum into slot r of
    // every CTA's table, one cluster barrier, then everybody adds its own table.  Nobody reads remote shared memory, so no
    // CTA has to wait at the end of the kernel for peers that might still be reading from it.
    bool peers_running = false;
    auto cluster_total = [&](double mine, int slot) {
        mine = block_sum_d(mine, s_red);
        if (!peers_running) { cluster_wait(); peers_running = true; }      // the arrival of the kernel's first line: every CTA has started
        if (threadIdx.x < CS) cluster_store_f64(&s_all[slot][rank], threadIdx.x, mine);
        cluster_arrive();
        cluster_wait();
        double tot = 0.0;
        for (unsigned r = 0; r < CS; r++) tot += s_all[slot][r];
        return tot;
    };
    float scale;
    if (p.rms) {
        double s = 0.0;
#pragma unroll
        for (int j = 0; j < 8; j++) s += (double)(v[j] * v[j]);
        const float ms = (float)(cluster_total(s, 0) / (double)n);
        scale = 1.0f / sqrtf(ms + p.eps);
    } else {
        double s = 0.0;
#pragma unroll
        for (int j = 0; j < 8; j++) s += (double)v[j];
        const float mean = (float)(cluster_total(s, 0) / (double)n);
        double s2 = 0.0;
#pragma unroll
        for (int j = 0; j < 8; j++) { v[j] = v[j] - mean; s2 += (double)(v[j] * v[j]); }
        const float var = (float)(cluster_total(s2, 1) / (double)n);
        scale = 1.0f / sqrtf(var + p.eps);
    }
    PI_TL_MARK(2);
    float y[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        float r = __fmul_rn(v[j], scale);                              // separate roundings, as separate graph nodes give
        if (p.w) r = __fmul_rn(r, wv[j]);
        if (p.b) r = __fadd_rn(r, bv[j]);
        y[j] = r;
    }
    if (p.y) {
        float * out = p.y + (size_t)t * n + c;
        *reinterpret_cast<float4 *>(out)     = make_float4(y[0], y[1], y[2], y[3]);
        *reinterpret_cast<float4 *>(out + 4) = make_float4(y[4], y[5], y[6], y[7]);
    }
    if (p.act_type) emit_act8(p.act_type, p.act, t, n, (int)(c / 8), y, true);
    if (p.act2_type && p.act2_src == 1) emit_act8(p.act2_type, p.act2, t, n, (int)(c / 8), y, true);
    PI_TL_MARK(3);
    PI_TL_MARK(4);
}

int launch_norm(const NormArgs & a, cudaStream_t st) {
    if (a.T <= 0) return PI_OK;
    PI_REQUIRE(a.n % 8 == 0 && a.n <= (int64_t)NORM_CHUNKS * 1024 * 8, "norm: n=%lld must be a multiple of 8 and <= %d",
               (long long)a.n, NORM_CHUNKS * 1024 * 8);
    NormP p;
    p.x = a.x; p.n = a.n; p.rms = a.rms; p.eps = a.eps; p.w = a.w; p.b = a.b;
    p.partial = a.partial; p.n_groups = a.n_groups; p.T = a.T; p.residual = a.residual; p.residual2 = a.residual2; p.in_bias = a.in_bias; p.x_out = a.x_out;
    p.partial_stride = a.partial_stride; p.status = a.status;
    p.x_ranks = 1; p.x_rank = 0; p.x_index = 0; p.x_per_step = 1; p.x_slot = 0; p.x_wait = 0;
    p.x_mbox_local = nullptr; p.x_step = nullptr; p.x_extra = nullptr;
    for (int q = 0; q < PI_MAX_RANKS; q++) p.x_mbox[q] = nullptr;
    const bool xch = a.xch && a.xch->n_ranks > 1;
    if (xch) {
        const pi_exchange & x = *a.xch;
        PI_REQUIRE(x.n_ranks <= PI_MAX_RANKS && x.mailbox_local && x.epoch && a.status, "norm: exchange not configured");
        PI_REQUIRE((int64_t)a.T * a.n <= x.slot_floats, "norm: vector of %lld floats does not fit a mailbox slot", (long long)a.T * a.n);
        p.x_ranks = x.n_ranks; p.x_rank = x.rank_id; p.x_index = a.xch_index; p.x_per_step = a.xch_per_step;
        p.x_slot = x.slot_floats; p.x_wait = a.wait_cycles > 0 ? a.wait_cycles : 2000000000LL;       // about a second
        for (int q = 0; q < x.n_ranks; q++) p.x_mbox[q] = x.mailbox_peer[q];
        p.x_mbox_local = x.mailbox_local; p.x_step = x.epoch; p.x_extra = a.xch_extra;
    }
    p.y = a.y; p.act_type = a.act_type; p.act = a.act; p.act2_type = a.act2_type; p.act2 = a.act2; p.act2_src = a.act2_src;
    static int use_cluster = -1;
    if (use_cluster < 0) { const char * v = getenv("PI_NORM_CLUSTER"); use_cluster = !(v && v[0] == '0'); }
    if ((use_cluster || xch) && (a.x || a.partial)) {
        int cs = 0;
        for (int k = 8; k >= (xch ? 1 : 2); k /= 2) if (a.n % (k * 256) == 0 && a.n / k / 8 <= 256) { cs = k; break; }
        if (cs) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(a.T * cs); cfg.blockDim = dim3((unsigned)(a.n / cs / 8)); cfg.dynamicSmemBytes = 0; cfg.stream = st;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr; cfg.numAttrs = a.pdl ? 2 : 1;
            PI_CUDA(cudaLaunchKernelEx(&cfg, k_norm_cluster, p));
            return PI_OK;
        }
    }
    PI_REQUIRE(!xch, "norm: the exchange needs a vector length that is a multiple of 256 with at most 2048 values per slice (got %lld)", (long long)a.n);
    int threads = (int)((a.n / 8 + NORM_CHUNKS - 1) / NORM_CHUNKS);
    threads = min(1024, max(32, (threads + 31) / 32 * 32));
    if (threads <= 512) PI_CUDA(launch_k(k_norm<512>, dim3(a.T), dim3(threads), 0, st, a.pdl, p));
    else                PI_CUDA(launch_k(k_norm<1024>, dim3(a.T), dim3(threads), 0, st, a.pdl, p));
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// ggml_rope_custom, modes 0 and 2 (ggml.c:11163-11325), angles from a host-built table so that device and CPU path
// rotate by the same float cos / sin.  Products and sums are rounded separately, as the CPU build does.
__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, float & o0, float & o1) {
    o0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    o1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

__global__ void k_rope(float * __restrict__ x, int n_heads, int head_dim, const int32_t * __restrict__ pos,
                       const float * __restrict__ cs, int neox) {
    const int t = blockIdx.y;
    const int half = head_dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;           // pair index over heads
    if (i >= n_heads * half) return;
    const int h = i / half, k = i - h * half;
    const float2 a = reinterpret_cast<const float2 *>(cs)[(size_t)pos[t] * half + k];
    float * v = x + ((size_t)t * n_heads + h) * head_dim;
    const int i0 = neox ? k : 2 * k, i1 = neox ? k + half : 2 * k + 1;
    float o0, o1;
    rope_pair(v[i0], v[i1], a.x, a.y, o0, o1);
    v[i0] = o0; v[i1] = o1;
}

int launch_rope(float * x, int T, int n_heads, int head_dim, const int32_t * pos, const float * cs, int neox, cudaStream_t st) {
    if (T <= 0) return PI_OK;
    const int pairs = n_heads * head_dim / 2;
    const dim3 grid((pairs + 255) / 256, T);
    k_rope<<<grid, 256, 0, st>>>(x, n_heads, head_dim, pos, cs, neox);
    PI_LAUNCH_CHECK("k_rope");
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// llm_build_kv_store + llm_build_kqv for one new token per sequence (llama.cpp:4383-4418, 4764-4850).
// One CTA per (query head, token).  Optional fused RoPE of q and k (cs != nullptr).  The first query head of each KV
// group stores the new K (after RoPE) and V as FP16; every head reads the new token's K/V from the F32 inputs
// (rounded to FP16, exactly what was stored) so no CTA depends on another one's store.
// CPU-path numerics: q and the probabilities are rounded to FP16 before the dot products; exp() goes through FP16
// in and out (the reference uses a table of FP16(expf(FP16))); the normaliser is summed in double.
// Latency-bound (the whole KV of a layer is ~1 MB): the score pass gives every thread one cached position and issues
// its head_dim/8 128-bit loads back to back; the value pass splits positions over ATTN_THREADS/(head_dim/8) slices.
static constexpr int ATTN_THREADS = 512;

struct AttnP {
    const float * q; const float * k; const float * v; __half * k_cache; __half * v_cache;
    const int32_t * seq; const int32_t * pos; int n_head, n_head_kv, hd, n_ctx;
    const float * cs; int neox; int sc_floats; int64_t q_stride, kv_stride;
    float * out; ActBuf out_act; int out_act_type; int store_mode;
};

__device__ __forceinline__ float dot8(const uint4 kv, const float * __restrict__ q) {
    const float2 k0 = h2f(kv.x), k1 = h2f(kv.y), k2 = h2f(kv.z), k3 = h2f(kv.w);
    float a = k0.x * q[0];
    a = fmaf(k0.y, q[1], a); a = fmaf(k1.x, q[2], a); a = fmaf(k1.y, q[3], a);
    a = fmaf(k2.x, q[4], a); a = fmaf(k2.y, q[5], a); a = fmaf(k3.x, q[6], a); a = fmaf(k3.y, q[7], a);
    return a;
}

__global__ void __launch_bounds__(ATTN_THREADS) k_attention(const AttnP p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ double s_red[ATTN_THREADS / 32];
    __shared__ float s_max[ATTN_THREADS / 32];
    const int h = blockIdx.x, t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int hd = p.hd, half = hd / 2, chunks = hd / 8;
    const int group = p.n_head / p.n_head_kv, hk = h / group;
    const int dkv = p.n_head_kv * hd;
    pdl_launch();
    // ---- before the wait: everything that no kernel of this step writes.  The position is set between steps and the
    //      cache rows below it were stored by earlier steps, so their loads (the long latency chain of this kernel)
    //      overlap the tail of the QKV mat-vec.
    const int pos = p.pos[t];
    const int sq = p.seq ? p.seq[t] : 0;
    if (pos < 0 || pos >= p.n_ctx) return;                       // never index the cache out of range
    __half * kc = p.k_cache + (size_t)sq * p.n_ctx * dkv + (size_t)hk * hd;
    __half * vc = p.v_cache + (size_t)sq * p.n_ctx * dkv + (size_t)hk * hd;
    const int slices = ATTN_THREADS / chunks;
    const int c8 = tid % chunks, sl = tid / chunks;
    // L2 prefetch hints cost no registers, so this CTA still fits beside the mat-vec CTAs it overlaps with
    for (int j = tid; j < pos && p.store_mode == 0; j += ATTN_THREADS) {
        const char * kr = reinterpret_cast<const char *>(kc + (size_t)j * dkv);
        const char * vr = reinterpret_cast<const char *>(vc + (size_t)j * dkv);
        for (int o = 0; o < hd * 2; o += 128) {
            asm volatile("prefetch.global.L2 [%0];" :: "l"(kr + o));
            asm volatile("prefetch.global.L2 [%0];" :: "l"(vr + o));
        }
    }
    float2 cs_reg = make_float2(1.f, 0.f);
    if (p.cs && tid < half) cs_reg = reinterpret_cast<const float2 *>(p.cs)[(size_t)pos * half + tid];
    pdl_wait();

    float *  sc  = reinterpret_cast<float *>(smem_raw);          // scores, then exp values, then the output slices
    float *  q32 = sc + p.sc_floats;                             // [hd] q rounded to FP16, widened
    __half * k16 = reinterpret_cast<__half *>(q32 + hd);         // [hd] the new token's K
    __half * v16 = k16 + hd;                                     // [hd] the new token's V
    __half * p16 = v16 + hd;                                     // [n_ctx] probabilities in FP16

    const float * qh = p.q + (size_t)t * p.q_stride + (size_t)h * hd;
    const float * kh = p.k + (size_t)t * p.kv_stride + (size_t)hk * hd;
    const float * vh = p.v + (size_t)t * p.kv_stride + (size_t)hk * hd;
    for (int e = tid; e < hd; e += ATTN_THREADS) v16[e] = __float2half_rn(vh[e]);
    if (p.cs) {
        if (tid < half) {                                        // half <= 128 < ATTN_THREADS
            const int k = tid;
            const int i0 = p.neox ? k : 2 * k, i1 = p.neox ? k + half : 2 * k + 1;
            float o0, o1;
            rope_pair(qh[i0], qh[i1], cs_reg.x, cs_reg.y, o0, o1);
            q32[i0] = round_f16(o0); q32[i1] = round_f16(o1);
            rope_pair(kh[i0], kh[i1], cs_reg.x, cs_reg.y, o0, o1);
            k16[i0] = __float2half_rn(o0); k16[i1] = __float2half_rn(o1);
        }
    } else {
        for (int e = tid; e < hd; e += ATTN_THREADS) { q32[e] = round_f16(qh[e]); k16[e] = __float2half_rn(kh[e]); }
    }
    __syncthreads();
    if (h % group == 0 && p.store_mode != 2) {
        for (int e = tid; e < hd; e += ATTN_THREADS) {
            kc[(size_t)pos * dkv + e] = k16[e];
            vc[(size_t)pos * dkv + e] = v16[e];
        }
    }
    if (p.store_mode == 1) return;                              // store pass of a prompt chunk

    PI_TL_MARK(0);
    // ---- scores.  head_dim/8 a power of two <= 32 (head_dim 32, 64, 128, 256): a group of head_dim/8 lanes reads one
    //      cached row as ONE coalesced request (a lane per 16-byte chunk, its 8 query values in registers), U rows in flight
    //      per group, the dot finished by a shuffle tree.  (One thread per row, the other branch, makes every request touch
    //      32 different rows and needs head_dim/32 dependent batches.)  The new token's K comes from shared memory.
    const float scale = 1.0f / sqrtf((float)hd);
    float mx = -INFINITY;
    if ((chunks & (chunks - 1)) == 0 && chunks <= 32) {
        constexpr int U = 12;                                        // rows in flight per group: 384 positions per round trip at head_dim 128
        const int LP = chunks, NG = ATTN_THREADS / LP, gi = tid / LP, c = tid % LP;
        float qr[8];
#pragma unroll
        for (int j = 0; j < 8; j++) qr[j] = q32[c * 8 + j];
        const int n_iter = (pos + NG) / NG;                          // ceil((pos + 1) / NG): the same for every lane
        for (int it = 0; it < n_iter; it += U) {
            uint4 kv[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = gi + (it + u) * NG;
                kv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (j < pos) kv[u] = __ldg(reinterpret_cast<const uint4 *>(kc + (size_t)j * dkv) + c);
                else if (j == pos) kv[u] = reinterpret_cast<const uint4 *>(k16)[c];
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = gi + (it + u) * NG;
                float a = dot8(kv[u], qr);
                for (int o = LP >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                a *= scale;
                if (c == 0 && j <= pos) { sc[j] = a; mx = fmaxf(mx, a); }
            }
        }
    } else {
        for (int j = tid; j <= pos; j += ATTN_THREADS) {
            float a = 0.f;
            if (j < pos) {
                const uint4 * kr = reinterpret_cast<const uint4 *>(kc + (size_t)j * dkv);
                float part[4] = {0.f, 0.f, 0.f, 0.f};
                for (int c = 0; c < chunks; c += 4) {
                    uint4 kv[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) kv[u] = __ldg(kr + c + u);               // chunks % 4 == 0 (head_dim % 32 == 0)
#pragma unroll
                    for (int u = 0; u < 4; u++) part[u] += dot8(kv[u], q32 + (c + u) * 8);
                }
                a = (part[0] + part[1]) + (part[2] + part[3]);
            } else {
                for (int c = 0; c < chunks; c++) a += dot8(reinterpret_cast<const uint4 *>(k16)[c], q32 + c * 8);
            }
            a *= scale;
            sc[j] = a;
            mx = fmaxf(mx, a);
        }
    }
    mx = warp_max(mx);
    if (lane == 0) s_max[wid] = mx;
    __syncthreads();
    mx = s_max[0];
#pragma unroll
    for (int i = 1; i < ATTN_THREADS / 32; i++) mx = fmaxf(mx, s_max[i]);

    PI_TL_MARK(1);
    // ---- softmax (ggml.c:10708-10777)
    double part = 0.0;
    for (int j = tid; j <= pos; j += ATTN_THREADS) {
        const float arg = round_f16(sc[j] - mx);
        const float e = round_f16(expf(arg));
        sc[j] = e;
        part += (double)e;
    }
    part = warp_sum_d(part);
    if (lane == 0) s_red[wid] = part;
    __syncthreads();
    {
        double tot = 0.0;
        for (int i = 0; i < ATTN_THREADS / 32; i++) tot += s_red[i];
        const float inv = (float)(1.0 / tot);
        for (int j = tid; j <= pos; j += ATTN_THREADS) p16[j] = __float2half_rn(sc[j] * inv);
    }
    __syncthreads();

    PI_TL_MARK(2);
    // ---- out[e] = sum_j p_j V[j, e]: thread = (chunk of 8 columns, slice of positions); slices reduced through smem
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    auto fma8 = [&](float pj, const uint4 vv) {
        const float2 v0 = h2f(vv.x), v1 = h2f(vv.y), v2 = h2f(vv.z), v3 = h2f(vv.w);
        acc[0] = fmaf(pj, v0.x, acc[0]); acc[1] = fmaf(pj, v0.y, acc[1]);
        acc[2] = fmaf(pj, v1.x, acc[2]); acc[3] = fmaf(pj, v1.y, acc[3]);
        acc[4] = fmaf(pj, v2.x, acc[4]); acc[5] = fmaf(pj, v2.y, acc[5]);
        acc[6] = fmaf(pj, v3.x, acc[6]); acc[7] = fmaf(pj, v3.y, acc[7]);
    };
    if (sl < slices) {
        constexpr int UV = 12;
        for (int j0 = sl; j0 <= pos; j0 += slices * UV) {
            uint4 vv[UV]; float pj[UV];
#pragma unroll
            for (int u = 0; u < UV; u++) {
                const int j = j0 + u * slices;
                pj[u] = 0.f; vv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (j <= pos) {
                    pj[u] = __half2float(p16[j]);
                    vv[u] = j == pos ? reinterpret_cast<const uint4 *>(v16)[c8]
                                     : __ldg(reinterpret_cast<const uint4 *>(vc + (size_t)j * dkv) + c8);
                }
            }
#pragma unroll
            for (int u = 0; u < UV; u++) fma8(pj[u], vv[u]);
        }
    }
    PI_TL_MARK(3);
    float * red = sc;                                              // exp values are dead: reuse as [slices][hd]
    if (sl < slices) {
#pragma unroll
        for (int j = 0; j < 8; j++) red[sl * hd + c8 * 8 + j] = acc[j];
    }
    __syncthreads();
    for (int e = tid; e < hd; e += ATTN_THREADS) {
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        int s2 = 0;
        for (; s2 + 4 <= slices; s2 += 4) {                         // 4 independent chains, joined in a fixed order
#pragma unroll
            for (int u = 0; u < 4; u++) o[u] += red[(s2 + u) * hd + e];
        }
        for (; s2 < slices; s2++) o[0] += red[s2 * hd + e];
        const float ov = (o[0] + o[1]) + (o[2] + o[3]);
        if (p.out) p.out[((size_t)t * p.n_head + h) * hd + e] = ov;
        red[e] = ov;                                               // slice 0 row now holds the final value (own column only)
    }
    if (p.out_act_type) {
        __syncthreads();
        // hd % 32 == 0: this head owns whole Q8 blocks of the concatenated [n_head*hd] vector
        const int64_t n = (int64_t)p.n_head * hd;
        if (wid == 0) {                                             // hd/8 <= 32 chunks: one per lane of warp 0
            const bool valid = lane < hd / 8;
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; j++) y[j] = valid ? red[lane * 8 + j] : 0.f;
            emit_act8(p.out_act_type, p.out_act, t, n, h * (hd / 8) + lane, y, valid);
        }
    }
    PI_TL_MARK(4);
}

int launch_attention(const AttnArgs & a, cudaStream_t st) {
    if (a.T <= 0) return PI_OK;
    PI_REQUIRE(a.head_dim % 32 == 0 && a.head_dim <= 256, "attention: head_dim=%d must be a multiple of 32, <= 256", a.head_dim);
    PI_REQUIRE(a.n_head % a.n_head_kv == 0, "attention: n_head %% n_head_kv != 0");
    AttnP p;
    p.q = a.q; p.k = a.k; p.v = a.v; p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.seq = a.seq; p.pos = a.pos;
    p.n_head = a.n_head; p.n_head_kv = a.n_head_kv; p.hd = a.head_dim; p.n_ctx = a.n_ctx;
    p.q_stride = a.q_stride ? a.q_stride : (int64_t)a.n_head * a.head_dim;
    p.kv_stride = a.kv_stride ? a.kv_stride : (int64_t)a.n_head_kv * a.head_dim;
    p.cs = a.cs; p.neox = a.neox; p.out = a.out; p.out_act = a.out_act; p.out_act_type = a.out_act_type; p.store_mode = a.store_mode;
    // sc must hold max(n_ctx, slices*hd) floats
    const int slices = ATTN_THREADS / (a.head_dim / 8);
    const size_t sc_floats = (size_t)((max(a.n_ctx, slices * a.head_dim) + 3) / 4 * 4);
    const size_t smem = sc_floats * 4 + (size_t)a.head_dim * 4 + (size_t)2 * a.head_dim * 2 + (size_t)a.n_ctx * 2 + 16;
    p.sc_floats = (int)sc_floats;
    static bool attr_set[16] = {false};
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    if (smem > 48 * 1024 && !(dev < 16 && attr_set[dev])) {
        PI_CUDA(cudaFuncSetAttribute(k_attention, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev < 16) attr_set[dev] = true;
    }
    PI_REQUIRE(smem <= 200 * 1024, "attention: n_ctx=%d needs %zu bytes of shared memory", a.n_ctx, smem);
    const dim3 grid(a.n_head, a.T);
    PI_CUDA(launch_k(k_attention, grid, dim3(ATTN_THREADS), smem, st, a.pdl, p));
    return PI_OK;
}

}  // namespace pi
