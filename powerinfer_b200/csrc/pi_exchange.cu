// Exchange of the per-layer partial d_model vectors between the ranks of one node (attention out-projection and FFN
// down-projection partials), fused with the reduction over the axpy's row groups that precedes it.
//
// One-shot push: each rank sums its own row-group partials and writes the result with plain 128-bit stores into slot
// `rank_id` of EVERY rank's mailbox (its own included), then raises that slot's flag to the new epoch with a
// system-scope release store.  The consumer (the norm kernel that follows) waits, with a bound, for the n_ranks flags
// of ITS OWN mailbox and adds the slots in rank order, so every rank computes bit-identical sums.  Nothing ever reads
// another GPU's memory, and no bulk / TMA / multicast copy is involved: only st.global over NVLink.
// Slots are double-buffered by epoch parity: a rank can be at most one exchange ahead of a peer, because it cannot
// finish exchange k before every peer has pushed k, which a peer does only after it has consumed k-1.
#include "pi_common.cuh"
#include <cstring>

namespace pi {

static constexpr int PUSH_WARPS = 32;

struct PushP {
    const float * partial; int n_groups; int64_t group_stride; int64_t total; const float * extra;
    float * mbox[PI_MAX_RANKS]; unsigned int * flags[PI_MAX_RANKS];
    int n_ranks, rank_id; int64_t slot_floats; unsigned int * epoch; unsigned int * ticket;
};

// A CTA owns 128 consecutive values.  Warp w adds groups w, w+32, ... (all its loads in flight at once: the partials
// were just written, so this is one L2 round trip, not n_groups of them); the 32 warp sums are added in warp order, then
// warp 0 stores the result into every rank's mailbox.  The order is fixed, so every launch gives the same bits.
__global__ void __launch_bounds__(PUSH_WARPS * 32) k_exchange_push(const PushP p) {
    __shared__ float4 s_part[PUSH_WARPS][32];
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    pdl_launch();
    pdl_wait();
    // every CTA reads the epoch before it takes a ticket; only the last ticket holder advances it
    const unsigned int e = *reinterpret_cast<volatile unsigned int *>(p.epoch) + 1u;
    const size_t slot = ((size_t)(e & 1u) * p.n_ranks + p.rank_id) * (size_t)p.slot_floats;
    const int64_t i4 = (int64_t)blockIdx.x * 32 + lane;                // float4 index
    const bool ok = i4 * 4 < p.total;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
        for (int j0 = w; j0 < p.n_groups; j0 += PUSH_WARPS * 8) {
            float4 a[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int j = j0 + u * PUSH_WARPS;
                a[u] = j < p.n_groups ? __ldcg(reinterpret_cast<const float4 *>(p.partial + (size_t)j * p.group_stride) + i4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) { v.x += a[u].x; v.y += a[u].y; v.z += a[u].z; v.w += a[u].w; }
        }
    }
    s_part[w][lane] = v;
    __syncthreads();
    if (w == 0 && ok) {
#pragma unroll
        for (int k = 1; k < PUSH_WARPS; k++) { const float4 a = s_part[k][lane]; v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w; }
        if (p.extra) {
            const float4 a = reinterpret_cast<const float4 *>(p.extra)[i4];
            v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
        }
        for (int q = 0; q < p.n_ranks; q++) reinterpret_cast<float4 *>(p.mbox[q] + slot)[i4] = v;
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (threadIdx.x < (unsigned)p.n_ranks) {
        unsigned int * f = p.flags[threadIdx.x] + (size_t)(e & 1u) * p.n_ranks + p.rank_id;
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(f), "r"(e) : "memory");
    }
    if (threadIdx.x == 0) { *p.epoch = e; *p.ticket = 0u; }
}

int launch_exchange_push(const pi_exchange & x, const float * partial, int n_groups, int T, int64_t n, const float * extra,
                         unsigned int * status, cudaStream_t st, bool pdl) {
    (void)status;
    PI_REQUIRE(x.n_ranks >= 1 && x.n_ranks <= PI_MAX_RANKS && x.mailbox_local && x.epoch && x.ticket, "exchange: not configured");
    PI_REQUIRE((int64_t)T * n <= x.slot_floats && (T * n) % 4 == 0, "exchange: vector of %lld floats does not fit a slot", (long long)T * n);
    PushP p;
    p.partial = partial; p.n_groups = n_groups; p.group_stride = (int64_t)T * n; p.total = (int64_t)T * n; p.extra = extra;
    for (int q = 0; q < PI_MAX_RANKS; q++) { p.mbox[q] = q < x.n_ranks ? x.mailbox_peer[q] : nullptr; p.flags[q] = q < x.n_ranks ? x.flags_peer[q] : nullptr; }
    p.n_ranks = x.n_ranks; p.rank_id = x.rank_id; p.slot_floats = x.slot_floats; p.epoch = x.epoch; p.ticket = x.ticket;
    const int grid = (int)((p.total / 4 + 31) / 32);
    PI_CUDA(launch_k(k_exchange_push, dim3(grid), dim3(PUSH_WARPS * 32), 0, st, pdl, p));
    return PI_OK;
}

}  // namespace pi

using namespace pi;

extern "C" {
#pragma GCC visibility push(default)

int pi_device_malloc(void ** ptr, size_t bytes) {
    PI_REQUIRE(ptr && bytes > 0, "device_malloc: bad arguments");
    PI_CUDA(cudaMalloc(ptr, bytes));
    PI_CUDA(cudaMemset(*ptr, 0, bytes));
    return PI_OK;
}
int pi_device_free(void * ptr) { PI_CUDA(cudaFree(ptr)); return PI_OK; }

int pi_ipc_export(void * ptr, void * host_handle64) {
    PI_REQUIRE(ptr && host_handle64, "ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    PI_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t *)host_handle64, ptr));
    return PI_OK;
}
int pi_ipc_import(const void * host_handle64, void ** ptr) {
    PI_REQUIRE(ptr && host_handle64, "ipc_import: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, host_handle64, sizeof h);
    PI_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return PI_OK;
}
int pi_ipc_close(void * ptr) { PI_CUDA(cudaIpcCloseMemHandle(ptr)); return PI_OK; }

#pragma GCC visibility pop
}
