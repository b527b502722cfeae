"""Whole-model parity at the PER-LAYER SHAPES of the benchmarked configurations: two-layer models with the layer shape of
the 7B-shape FP16 model (d 4096, F 11008, 32 heads), the falcon-40B-shape model (d 8192, F 32768, 128 / 8 heads of 64, two
layer norms, parallel block), the 70B-shape Q4_0 model (d 8192, F 28672, 64 / 8 heads, FP16 predictors) and the
opt-175B-shape model (d 12288, F 49152, rank-1536 predictors, learned positions), vocabulary cut to 1024 rows.  The golden
logits and greedy ids come from the reference's own llama.cpp run of the same files (one thread).  Bars as stated for the
path: FP16 logits within 2e-2, Q4_0 within 5e-2 (teacher-forced, 32 steps), active sets identical outside 1e-3 of the
threshold, free-running greedy stream identical for 32 tokens."""
import os

import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import synth
from test_gpu_engine import GOLD, check_teacher_forced

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def engine_mod():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import engine
    return engine


@pytest.mark.parametrize("name", sorted(mg.SHAPE_CASES))
def test_configuration_shaped_model_teacher_forced_and_free_running_32_tokens(engine_mod, name):
    spec = mg.SHAPE_CASES[name]
    g = np.load(os.path.join(GOLD, f"model_{name}.npz"))
    tensors = synth.build_model(spec)                           # drawn once for both halves (the large ones take a minute)
    worst, flip_steps = check_teacher_forced(engine_mod, name, practice_bar=5e-2 if spec.wtype == synth.Q4_0 else 2e-2, tensors=tensors)
    print(f"{name}: max |logit error| {worst:.2e} over the steps whose active sets agree, {flip_steps} steps with a borderline flip")
    eng = engine_mod.DecodeEngine(spec, tensors, max_batch=1)
    toks = [int(v) for v in g["prompt"]]
    for pos, tk in enumerate(toks[:-1]):
        eng.decode([tk], [pos], want_logits=False)
    cur, pos, stream = toks[-1], len(toks) - 1, []
    for _ in range(mg.N_STEPS):
        cur = int(eng.decode([cur], [pos], want_logits=False)[1][0])
        stream.append(cur)
        pos += 1
    eng.status()
    eng.close()
    assert mg.N_STEPS >= 32 and stream == [int(v) for v in g["greedy"]]
