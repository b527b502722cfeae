// ggml_axpy for callers that are not allowed to allocate device memory.
//
// Some hosts of this library hand out device memory themselves and forbid a plug-in to call cudaMalloc (an inference
// server with a fixed arena, a process that has already given all of HBM to its weight pool), and some call sites simply
// have no buffer at hand (code that runs while a stream is being captured, where an allocation is not permitted).
// pi_axpy needs scratch (active list, ticket words, partial sums); pi_axpy_static is the same operator with that scratch
// taken from a fixed array that lives in the library's own device image, so nothing is allocated, ever.
#include "pi_common.cuh"

namespace pi {

// Scratch of pi_axpy_static.  It is part of the loaded module: every GPU that loads the library holds these bytes until the
// process exits.  In host code this name is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress below.
static constexpr size_t STATIC_AXPY_BYTES = (size_t)24 << 20;
static __device__ __align__(256) unsigned char g_axpy_scratch[STATIC_AXPY_BYTES];

static constexpr int MAX_DEVICES = 64;
static void * g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the CURRENT device; looked up once per device.
int static_scratch_address(void ** out) {
    int dev = 0;
    PI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) { set_error("axpy_static: device ordinal %d not supported", dev); return PI_ERR_UNSUPPORTED; }
    if (!g_scratch_ptr[dev]) {
        void * p = nullptr;
        PI_CUDA(cudaGetSymbolAddress(&p, g_axpy_scratch));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return PI_OK;
}

}  // namespace pi

using namespace pi;

extern "C" {
#pragma GCC visibility push(default)

size_t pi_axpy_static_max_bytes(void) { return STATIC_AXPY_BYTES; }

int pi_axpy_static(int wtype, const void * Wt, int64_t n_w_rows, int64_t ncols,
                   const float * h, int64_t h_stride, const float * idx, int64_t idx_stride,
                   const int32_t * bucket, float threshold, float * dst, void * stream) {
    // limits first, so that an oversized request fails the same way on every device and before any CUDA call
    PI_REQUIRE(n_w_rows >= 0 && n_w_rows <= 65536 && h_stride <= 65536 && ncols > 0 && ncols <= 16384,
               "axpy_static: one token, at most 65536 neurons and 16384 columns (got %lld rows, h_stride %lld, %lld columns); "
               "use pi_axpy with a caller-provided workspace for larger shapes",
               (long long)n_w_rows, (long long)h_stride, (long long)ncols);
    const size_t need = pi_workspace_bytes(ncols, n_w_rows > h_stride ? n_w_rows : h_stride, 1);
    PI_REQUIRE(need <= STATIC_AXPY_BYTES, "axpy_static: this shape needs %zu bytes of scratch, the built-in array holds %zu; use pi_axpy",
               need, STATIC_AXPY_BYTES);
    void * scratch = nullptr;
    const int rc = static_scratch_address(&scratch);
    if (rc) return rc;
    // pi_axpy clears the words that must start at zero (count, ticket, status) itself and overwrites the rest before
    // reading it, so whatever the previous call left in the array is harmless.
    return pi_axpy(wtype, Wt, n_w_rows, ncols, h, 1, h_stride, idx, idx_stride, bucket, threshold, dst, scratch, STATIC_AXPY_BYTES, stream);
}

#pragma GCC visibility pop
}
