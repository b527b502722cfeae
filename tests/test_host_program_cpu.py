"""powerinfer_b200/host/pi_decode.cpp (a C++ program that decodes through the C ABI alone) compiles and links against the
header and the library, reads a model file with the native reader and reports its configuration; without a device it stops
at its first CUDA call with a message and exit code 1 (there is no CPU path to fall back to).  Its output on a GPU is
checked in tests/test_gpu_host_program.py."""
import os
import shutil
import subprocess

import pytest

import make_golden as mg
from powerinfer_b200 import _lib, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def compile_pi_decode(out_dir):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    lib = _lib.LIB_PATH                     # the library as built (importing the package fails loudly when it is missing)
    exe = os.path.join(str(out_dir), "pi_decode")
    libdir = os.path.dirname(lib)
    r = subprocess.run([nvcc, "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", os.path.join(ROOT, "include"),
                        os.path.join(ROOT, "powerinfer_b200", "host", "pi_decode.cpp"), "-L", libdir, "-lpowerinfer_b200",
                        "-Xlinker", "-rpath", "-Xlinker", libdir, "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return exe


def test_host_program_reads_the_model_and_fails_cleanly_without_a_device(tmp_path):
    pytest.importorskip("gguf")
    torch = pytest.importorskip("torch")
    exe = compile_pi_decode(tmp_path)
    spec = mg.MODEL_CASES["llama_q4_0"]
    path = str(tmp_path / "m.powerinfer.gguf")
    mg.write_gguf(spec, synth.build_model(spec), path)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 2 and "usage" in r.stderr
    r = subprocess.run([exe, str(tmp_path / "missing.gguf"), "4", "5"], capture_output=True, text=True)
    assert r.returncode == 1 and "cannot open" in r.stderr
    r = subprocess.run([exe, path, "4", "99999"], capture_output=True, text=True)
    assert r.returncode == 1 and "vocabulary" in r.stderr
    r = subprocess.run([exe, path, "4000", "5"], capture_output=True, text=True)
    assert r.returncode == 1 and "context length" in r.stderr
    r = subprocess.run([exe, path, "4", "5", "6"], capture_output=True, text=True)
    want = (f"model: arch=llama weights=q4_0 layers={spec.n_layer} d={spec.d} ff={spec.n_ff} heads={spec.n_head}/{spec.n_head_kv} "
            f"rank={spec.rank} vocab={spec.n_vocab} ctx={spec.n_ctx}")
    assert want in r.stdout, r.stdout
    if not torch.cuda.is_available():
        assert r.returncode == 1 and "CUDA" in r.stderr and "ids:" not in r.stdout
