"""The bamboo architecture on the GPU: the llama graph with the symmetric gate h = relu(gate) * relu(up)
(LLM_FFN_SYM, llama.cpp:4732-4738, 5028).  The engine gets it from the gated mat-vec's relu-on-output switch, since
relu(gate) * relu(up) == relu(relu(gate) * up) exactly when the first factor is non-negative.  Checked like the other
architectures: teacher-forced logits and the greedy stream against the reference's llama.cpp run of a `bamboo` model file
(golden fixture), the active sets against the CPU checker, a batch against single sequences, and the file loader."""
import os

import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import synth
from test_gpu_engine import GOLD, check_batched_vs_single, check_teacher_forced

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def engine_mod():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import engine
    return engine


def test_bamboo_teacher_forced_logits_and_greedy_stream(engine_mod):
    check_teacher_forced(engine_mod, "bamboo_f16")


def test_bamboo_batched_sequences_match_single(engine_mod):
    check_batched_vs_single(engine_mod, "bamboo_f16", 4)


def test_bamboo_differs_from_the_parallel_gate(engine_mod):
    """The same weights run as plain llama must NOT reproduce the bamboo fixture: the switch is live."""
    import dataclasses
    spec = mg.MODEL_CASES["bamboo_f16"]
    g = np.load(os.path.join(GOLD, "model_bamboo_f16.npz"))
    t = synth.build_model(spec)
    out = {}
    for sym in (True, False):
        eng = engine_mod.DecodeEngine(dataclasses.replace(spec, gate_sym=sym), t, max_batch=1)
        for pos, tk in enumerate(int(v) for v in g["prompt"]):
            logits, _ = eng.decode([tk], [pos])
        out[sym] = logits[0].copy()
        eng.close()
    assert np.abs(out[True] - g["logits"][0]).max() <= 2e-2
    assert np.abs(out[False] - g["logits"][0]).max() > 5e-2


def test_bamboo_model_file_loads_as_symmetric_gate(engine_mod, tmp_path):
    pytest.importorskip("gguf")
    from powerinfer_b200 import gguf_loader
    spec = mg.MODEL_CASES["bamboo_f16"]
    path = str(tmp_path / "bamboo.powerinfer.gguf")
    mg.write_gguf(spec, synth.build_model(spec), path)
    spec2, t2 = gguf_loader.load_model(path)
    assert spec2.gate_sym and spec2.arch == synth.ARCH_LLAMA
    g = np.load(os.path.join(GOLD, "model_bamboo_f16.npz"))
    eng = engine_mod.DecodeEngine(spec2, t2, max_batch=1)
    for pos, tk in enumerate(int(v) for v in g["prompt"]):
        logits, _ = eng.decode([tk], [pos])
    assert np.abs(logits[0] - g["logits"][0]).max() <= 2e-2
    eng.close()
