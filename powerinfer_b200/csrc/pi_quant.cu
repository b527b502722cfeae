// Block formats of the hot path: Q4_0 weights (quantise, re-layout, dequantise) and the Q8_0 / FP16
// forms activations take before a mat-vec.  All kernels are HBM- or latency-bound byte shuffles.
#include "pi_common.cuh"

namespace pi {

static constexpr int QK = 32;

// ------------------------------------------------------------------------------------------------
// quantize_row_q4_0_reference (ggml-quants.c:428-463).  One warp per block of 32 values, lane = value.
// The reference keeps the FIRST value of largest magnitude; ties are resolved to the lowest lane.
__global__ void k_quantize_q4_0(const float * __restrict__ x, uint8_t * __restrict__ q, int64_t nblocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += warps) {
        const float v = x[b * QK + lane];
        float amax = fabsf(v);
        int   arg  = lane;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
            const int   ol = __shfl_xor_sync(0xffffffffu, arg, o);
            if (oa > amax || (oa == amax && ol < arg)) { amax = oa; arg = ol; }
        }
        const float mx = __shfl_sync(0xffffffffu, v, arg);
        const float d  = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        // two roundings as in the reference (x*id, then +8.5): keep the compiler from fusing them into one FMA
        int qi = (int)(int8_t)__fadd_rn(__fmul_rn(v, id), 8.5f);   // float -> int8 truncates toward zero
        qi = qi > 15 ? 15 : qi;
        const int hi = __shfl_down_sync(0xffffffffu, qi, 16);
        uint8_t * blk = q + b * 18;
        if (lane == 0) *reinterpret_cast<__half *>(blk) = __float2half_rn(d);
        if (lane < 16) blk[2 + lane] = (uint8_t)((qi & 0xF) | (hi << 4));
    }
}

int launch_quantize_q4_0(const float * x, void * q4, int64_t nrows, int64_t ncols, cudaStream_t st) {
    const int64_t nblocks = nrows * (ncols / QK);
    if (nblocks == 0) return PI_OK;
    const int grid = (int)imin64((nblocks + 7) / 8, (int64_t)sm_count() * 16);
    k_quantize_q4_0<<<grid, 256, 0, st>>>(x, (uint8_t *)q4, nblocks);
    PI_LAUNCH_CHECK("k_quantize_q4_0");
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// ggml layout: row = nb x {fp16 d; uint8 qs[16]}.  Planar layout: row = nb x qs[16] then nb x fp16 d.
// One thread per block; 2-byte accesses on the ggml side (blocks are only 2-byte aligned).
__global__ void k_q4_0_repack(const uint8_t * __restrict__ src, uint8_t * __restrict__ dst, int64_t nrows, int nb) {
    const int64_t total = nrows * nb;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nb;
        const int b = (int)(i - r * nb);
        const uint16_t * s = reinterpret_cast<const uint16_t *>(src + (r * nb + b) * 18);
        uint8_t * row = dst + r * (int64_t)nb * 18;
        uint16_t w[9];
#pragma unroll
        for (int j = 0; j < 9; j++) w[j] = s[j];
        uint4 qv;
        qv.x = w[1] | ((uint32_t)w[2] << 16);
        qv.y = w[3] | ((uint32_t)w[4] << 16);
        qv.z = w[5] | ((uint32_t)w[6] << 16);
        qv.w = w[7] | ((uint32_t)w[8] << 16);
        reinterpret_cast<uint4 *>(row)[b] = qv;
        reinterpret_cast<uint16_t *>(row + (int64_t)nb * 16)[b] = w[0];
    }
}

int launch_q4_0_repack(const void * src, void * dst, int64_t nrows, int64_t ncols, cudaStream_t st) {
    const int nb = (int)(ncols / QK);
    const int64_t total = nrows * nb;
    if (total == 0) return PI_OK;
    const int grid = (int)imin64((total + 255) / 256, (int64_t)sm_count() * 16);
    k_q4_0_repack<<<grid, 256, 0, st>>>((const uint8_t *)src, (uint8_t *)dst, nrows, nb);
    PI_LAUNCH_CHECK("k_q4_0_repack");
    return PI_OK;
}

// dequantize_row_q4_0 (ggml-quants.c:1074-1092) from the planar layout; one thread per block
__global__ void k_dequantize_q4_0(const uint8_t * __restrict__ q, float * __restrict__ y, int64_t nrows, int nb) {
    const int64_t total = nrows * nb;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / nb;
        const int b = (int)(i - r * nb);
        const uint8_t * row = q + r * (int64_t)nb * 18;
        const uint4 qv = reinterpret_cast<const uint4 *>(row)[b];
        const float d = __half2float(reinterpret_cast<const __half *>(row + (int64_t)nb * 16)[b]);
        const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
        float * o = y + (r * nb + b) * QK;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const uint32_t byte = (w[j >> 2] >> ((j & 3) * 8)) & 0xFFu;
            o[j]      = (float)((int)(byte & 0xF) - 8) * d;
            o[j + 16] = (float)((int)(byte >> 4) - 8) * d;
        }
    }
}

int launch_dequantize_q4_0(const void * q4p, float * y, int64_t nrows, int64_t ncols, cudaStream_t st) {
    const int nb = (int)(ncols / QK);
    const int64_t total = nrows * nb;
    if (total == 0) return PI_OK;
    const int grid = (int)imin64((total + 255) / 256, (int64_t)sm_count() * 16);
    k_dequantize_q4_0<<<grid, 256, 0, st>>>((const uint8_t *)q4p, y, nrows, nb);
    PI_LAUNCH_CHECK("k_dequantize_q4_0");
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// quantize_row_q8_0, the AVX2 branch the CPU path runs (ggml-quants.c:702-760):
//   d = amax / 127, id = amax != 0 ? 127 / amax : 0, q = round-to-nearest-even(x * id), d stored as FP16.
// One warp per block, lane = value.
__device__ __forceinline__ void q8_block(float v, int & q, float & d16, int & sum) {
    const float amax = warp_max(fabsf(v));
    const float d  = amax / 127.0f;
    const float id = amax != 0.0f ? 127.0f / amax : 0.0f;
    q = __float2int_rn(v * id);
    d16 = __half2float(__float2half_rn(d));
    sum = warp_sum_i(q);
}

__global__ void k_quantize_q8_0_ggml(const float * __restrict__ x, uint8_t * __restrict__ q8, int64_t nblocks) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += warps) {
        int q, s; float d16;
        q8_block(x[b * QK + lane], q, d16, s);
        uint8_t * blk = q8 + b * 34;
        if (lane == 0) *reinterpret_cast<__half *>(blk) = __float2half_rn(d16);
        reinterpret_cast<int8_t *>(blk + 2)[lane] = (int8_t)q;
    }
}

int launch_quantize_q8_0_ggml(const float * x, void * q8, int64_t nrows, int64_t ncols, cudaStream_t st) {
    const int64_t nblocks = nrows * (ncols / QK);
    if (nblocks == 0) return PI_OK;
    const int grid = (int)imin64((nblocks + 7) / 8, (int64_t)sm_count() * 16);
    k_quantize_q8_0_ggml<<<grid, 256, 0, st>>>(x, (uint8_t *)q8, nblocks);
    PI_LAUNCH_CHECK("k_quantize_q8_0_ggml");
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// Activation planes (see Act in pi_common.cuh)
size_t act_bytes(int wtype, int64_t n, int T) {
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    if (wtype == PI_TYPE_Q4_0) {
        const size_t nb = (size_t)(n / QK);
        return 2 * up((size_t)T * nb * 16) + 2 * up((size_t)T * nb * 4);
    }
    return up((size_t)T * n * 2);
}

ActBuf act_carve(int wtype, int64_t n, int T, char ** p) {
    auto take = [&](size_t bytes) { char * r = *p; *p += (bytes + 255) & ~size_t(255); return r; };
    ActBuf a;
    if (wtype == PI_TYPE_Q4_0) {
        const size_t nb = (size_t)(n / QK);
        a.lo = (uint4 *)take((size_t)T * nb * 16);
        a.hi = (uint4 *)take((size_t)T * nb * 16);
        a.d  = (float *)take((size_t)T * nb * 4);
        a.s  = (int *)take((size_t)T * nb * 4);
    } else {
        a.h16 = (__half *)take((size_t)T * n * 2);
    }
    return a;
}

__global__ void k_act_f16(const float * __restrict__ x, int64_t x_stride, int64_t n, int T, __half * __restrict__ out) {
    const int64_t total = (int64_t)T * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n, c = i - t * n;
        out[i] = __float2half_rn(x[t * x_stride + c]);
    }
}

__global__ void k_act_q8(const float * __restrict__ x, int64_t x_stride, int nb, int T, ActBuf out) {
    const int lane = threadIdx.x & 31;
    const int64_t nblocks = (int64_t)T * nb;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < nblocks; i += warps) {
        const int64_t t = i / nb;
        const int b = (int)(i - t * nb);
        int q, s; float d16;
        q8_block(x[t * x_stride + (int64_t)b * QK + lane], q, d16, s);
        int8_t * plane = reinterpret_cast<int8_t *>(lane < 16 ? out.lo + i : out.hi + i);
        plane[lane & 15] = (int8_t)q;
        if (lane == 0) { out.d[i] = d16; out.s[i] = s; }
    }
}

int launch_convert_act(int wtype, const float * x, int64_t x_stride, int64_t n, int T, ActBuf out, cudaStream_t st) {
    if (T == 0 || n == 0) return PI_OK;
    if (wtype == PI_TYPE_Q4_0) {
        const int nb = (int)(n / QK);
        const int64_t nblocks = (int64_t)T * nb;
        const int grid = (int)imin64((nblocks + 7) / 8, (int64_t)sm_count() * 8);
        k_act_q8<<<grid, 256, 0, st>>>(x, x_stride, nb, T, out);
        PI_LAUNCH_CHECK("k_act_q8");
    } else {
        const int64_t total = (int64_t)T * n;
        const int grid = (int)imin64((total + 255) / 256, (int64_t)sm_count() * 8);
        k_act_f16<<<grid, 256, 0, st>>>(x, x_stride, n, T, out.h16);
        PI_LAUNCH_CHECK("k_act_f16");
    }
    return PI_OK;
}

// ------------------------------------------------------------------------------------------------
// Coefficients of the Q4_0 axpy (ggml.c:14575-14581): the FFN hidden vector quantised to Q8_0 over blocks of
// 32 consecutive NEURONS; neuron r contributes int8 b = cq[r] with scale cd[r/32].
__global__ void k_neuron_q8(const float * __restrict__ h, int64_t stride, int nb, int T,
                            int8_t * __restrict__ cq, float * __restrict__ cd) {
    const int lane = threadIdx.x & 31;
    const int64_t nblocks = (int64_t)T * nb;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t i = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < nblocks; i += warps) {
        const int64_t t = i / nb;
        const int b = (int)(i - t * nb);
        int q, s; float d16;
        q8_block(h[t * stride + (int64_t)b * QK + lane], q, d16, s);
        cq[t * stride + (int64_t)b * QK + lane] = (int8_t)q;
        if (lane == 0) cd[t * (stride / QK) + b] = d16;
    }
}

int launch_neuron_q8(const float * h, int64_t stride, int64_t n, int T, int8_t * cq, float * cd, cudaStream_t st) {
    const int nb = (int)(n / QK);
    const int64_t nblocks = (int64_t)T * nb;
    if (nblocks == 0) return PI_OK;
    const int grid = (int)imin64((nblocks + 7) / 8, (int64_t)sm_count() * 8);
    k_neuron_q8<<<grid, 256, 0, st>>>(h, stride, nb, T, cq, cd);
    PI_LAUNCH_CHECK("k_neuron_q8");
    return PI_OK;
}

}  // namespace pi
