"""The reference-side shim shown in INTEGRATION.md must compile against the reference's own ggml.h / ggml-cuda.h and
this library's header: field names, op enums and every argument list are checked by the compiler.  The few things the
snippet finds around it inside ggml-cuda.cu (streams, the tensor extra, the pool, the CUDA runtime calls) are declared
as stand-ins here.  Skipped where the reference tree is not present."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("PI_REFERENCE_DIR", "/root/reference")

STAND_INS = r"""
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include "ggml.h"
#include "ggml-cuda.h"
typedef struct CUstream_st * cudaStream_t;
enum cudaMemcpyKind { cudaMemcpyHostToDevice = 1 };
extern "C" int cudaMemcpyAsync(void *, const void *, size_t, cudaMemcpyKind, cudaStream_t);
extern "C" int cudaStreamSynchronize(cudaStream_t);
#define GGML_CUDA_MAX_DEVICES 16
#define MAX_STREAMS 8
static int g_main_device = 0;
static cudaStream_t g_cudaStreams[GGML_CUDA_MAX_DEVICES][MAX_STREAMS];
struct ggml_tensor_extra_gpu { void * data_device[GGML_CUDA_MAX_DEVICES]; };
static void * ggml_cuda_pool_malloc(size_t size, size_t * actual_size);
static void ggml_cuda_pool_free(void * ptr, size_t size);
static bool ggml_cuda_compute_forward_stock(struct ggml_compute_params * params, struct ggml_tensor * tensor);
extern float sparse_pred_threshold;
"""


def test_reference_side_shim_compiles_against_the_reference_headers(tmp_path):
    if not os.path.exists(os.path.join(REF, "ggml-cuda.h")) or shutil.which("g++") is None:
        pytest.skip("reference tree or g++ not present")
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    start = text.index("```cpp") + len("```cpp")
    code = text[start:text.index("```", start)]
    assert "ggml_cuda_compute_forward" in code and "pi_mul_mat_idx" in code and "pi_axpy" in code
    src = tmp_path / "shim.cpp"
    src.write_text(STAND_INS + code)
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-w", "-I", REF, "-I", os.path.join(ROOT, "include"), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
