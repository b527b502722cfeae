"""The drop-in back end without a GPU: libggml_cuda_b200.so must define every function the reference's ggml-cuda.h declares
and its host code calls, and the reference's host program linked against it must behave as the reference does when no
CUDA device is present: ggml_init_cublas succeeds, ggml_cublas_loaded is false, and the reference's own loader then
refuses a sparse model with "CUDA is not loaded" (llama.cpp:188-192): a clean refusal, not a crash in the back end."""
import ctypes as C
import os
import subprocess
import tempfile

import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import build, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "powerinfer_b200", "libggml_cuda_b200.so")
EXE = os.path.join(ROOT, "oracle", "_ref", "ref_decode_b200")

# ggml-cuda.h:14-64, minus debug_equal (declared there, defined nowhere in the reference)
SYMBOLS = """ggml_init_cublas ggml_cublas_loaded ggml_cuda_host_malloc ggml_cuda_host_free ggml_cuda_can_mul_mat
ggml_cuda_set_tensor_split ggml_cuda_transform_tensor ggml_cuda_alloc_tensor ggml_cuda_free_data ggml_cuda_cpy_1d
ggml_cuda_get_data_pp ggml_cuda_assign_buffers ggml_cuda_assign_buffers_no_scratch ggml_cuda_assign_buffers_force_inplace
ggml_cuda_assign_buffers_no_alloc ggml_cuda_assign_scratch_offset ggml_cuda_copy_to_device ggml_cuda_copy_to_host
ggml_cuda_set_main_device ggml_cuda_set_mul_mat_q ggml_cuda_set_scratch_size ggml_cuda_free_scratch
ggml_cuda_compute_forward ggml_cuda_get_device_count ggml_cuda_get_device_description ggml_cuda_get_free_memory
ggml_cuda_set_device_constants ggml_backend_cuda_init""".split()


def test_back_end_exports_the_ggml_cuda_h_symbol_set():
    if not os.path.exists(LIB):
        pytest.skip("libggml_cuda_b200.so was not built (needs the reference's headers at build time)")
    lib = C.CDLL(LIB)
    missing = [s for s in SYMBOLS if not hasattr(lib, s)]
    assert not missing, missing
    ref = build.reference_dir()
    if ref:                                                     # every GGML_API function of the header, read from the header itself
        import re
        text = open(os.path.join(ref, "ggml-cuda.h")).read()
        declared = set(re.findall(r"GGML_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)) - {"debug_equal"}
        assert declared <= set(SYMBOLS), declared - set(SYMBOLS)


def test_host_program_over_the_back_end_without_a_device_is_refused_by_the_reference_loader():
    if not os.path.exists(EXE):
        pytest.skip("oracle/_ref/ref_decode_b200 was not built")
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a CUDA device is present: covered by the GPU test")
    except ImportError:
        pass
    name = "llama_q4_0"
    spec = mg.MODEL_CASES[name]
    g = np.load(os.path.join(ROOT, "tests", "golden", f"model_{name}.npz"))
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, name + ".powerinfer.gguf")
        mg.write_gguf(spec, synth.build_model(spec), path)
        tp, op = os.path.join(td, "tok.i32"), os.path.join(td, "out.f32")
        np.asarray(g["prompt"], np.int32).tofile(tp)
        r = subprocess.run([EXE, path, tp, str(len(g["prompt"])), "4", "1", op, "single"], capture_output=True, text=True,
                           env=dict(os.environ, REF_VRAM_GB="0"), timeout=600)
    assert r.returncode == 1 and "CUDA is not loaded" in r.stderr, (r.returncode, r.stderr[-2000:])
    lib = C.CDLL(LIB)
    lib.ggml_cublas_loaded.restype = C.c_bool
    lib.ggml_init_cublas()
    assert lib.ggml_cublas_loaded() is False
