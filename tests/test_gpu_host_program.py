"""The C++ host program powerinfer_b200/host/pi_decode.cpp on a GPU: model file -> native reader -> uploads (Q4_0 through
pi_q4_0_repack, q / k / v stacked, falcon's fused matrix as stored) -> engine -> greedy ids, which must equal the
reference's llama.cpp stream for the same file and prompt (golden fixtures).  No Python touches the data path; this test
only writes the file and compares the printed ids."""
import os
import subprocess

import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import synth
from test_host_program_cpu import compile_pi_decode

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pytest.importorskip("gguf")
    return compile_pi_decode(tmp_path_factory.mktemp("pi_decode"))


@pytest.mark.parametrize("name", ["llama_f16", "llama_q4_0", "falcon_f16", "bamboo_f16"])
def test_cpp_host_program_reproduces_the_reference_greedy_stream(exe, tmp_path, name):
    spec = mg.MODEL_CASES[name]
    g = np.load(os.path.join(GOLD, f"model_{name}.npz"))
    path = str(tmp_path / "m.powerinfer.gguf")
    mg.write_gguf(spec, synth.build_model(spec), path)
    r = subprocess.run([exe, path, str(mg.N_STEPS)] + [str(int(t)) for t in g["prompt"]], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, (r.stdout[-500:], r.stderr[-2000:])
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("ids:")]
    assert line, r.stdout
    ids = [int(v) for v in line[0].split()[1:]]
    assert ids == [int(v) for v in g["greedy"]]
