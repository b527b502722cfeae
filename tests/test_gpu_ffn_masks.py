"""The one-token sparse FFN at the extremes of the activity mask, through the engine, against the CPU checker: every
neuron active (threshold far below every logit: each cluster of the single-launch FFN kernel then holds its largest
possible share of rows), no neuron active (the FFN contributes exactly its bias, every cluster writes a zero partial
vector), and half of them.  Shapes with a ragged last 1024-column slice and with fewer slices than a cluster has CTAs
are included.  The same cases run with the single-launch kernel switched off (child process), and both must agree with
the checker."""
import dataclasses
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import pio
from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BASE = {
    "llama_q4_0_d2048": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.Q4_0, n_layer=2, d=2048, n_ff=5632, n_head=16, n_head_kv=4, rank=128,
                                        firing=0.12, seed=51),
    "llama_f16_d1280": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, n_layer=2, d=1280, n_ff=3456, n_head=10, n_head_kv=10, rank=64,
                                       firing=0.2, seed=52),
    "opt_f16_d512": synth.ModelSpec(arch=synth.ARCH_OPT, wtype=synth.F16, n_layer=2, d=512, n_ff=2048, n_head=8, n_head_kv=8, rank=64,
                                    firing=0.15, seed=53, norm_eps=0.0),
    "falcon_q4_0_d1024": synth.ModelSpec(arch=synth.ARCH_FALCON, wtype=synth.Q4_0, n_layer=2, d=1024, n_ff=4096, n_head=16, n_head_kv=2, rank=64,
                                         firing=0.15, seed=54),
}
THRESHOLDS = {"all_active": -1e30, "none_active": 1e30, "model": None}


def run_case(name, which):
    from powerinfer_b200 import engine
    spec = BASE[name]
    if THRESHOLDS[which] is not None:
        spec = dataclasses.replace(spec, threshold=THRESHOLDS[which])
    t = synth.build_model(spec)
    eng = engine.DecodeEngine(spec, t, max_batch=1)
    eng.enable_trace()
    om = pio.OracleModel(spec, t)
    worst, cur = 0.0, 7
    for pos in range(6):
        logits, amax = eng.decode([cur], [pos])
        got = eng.predictor_trace(1)[:, 0]
        ref, pred = om.decode_imposed(cur, pos, got)
        n_active = int((got >= spec.threshold).sum())
        if which == "all_active":
            assert n_active == spec.n_layer * spec.n_ff
        if which == "none_active":
            assert n_active == 0
        worst = max(worst, float(np.abs(logits[0] - ref).max()))
        cur = int(ref.argmax())
    eng.status()
    eng.close()
    om.close()
    return worst


@pytest.mark.parametrize("which", sorted(THRESHOLDS))
@pytest.mark.parametrize("name", sorted(BASE))
def test_single_launch_ffn_mask_extremes(name, which):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    worst = run_case(name, which)
    bar = 5e-2 if BASE[name].wtype == synth.Q4_0 else 2e-2
    print(f"{name} / {which}: max |logit error| against the checker under identical active sets {worst:.2e} (bar {bar})")
    assert worst <= bar, worst


def test_two_kernel_path_same_cases():
    """PI_FFN_FUSED=0 (read when the library first plans a launch, hence a child process): gather and axpy as two launches."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    code = (f"import sys; sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {ROOT!r} + '/tests')\n"
            "import test_gpu_ffn_masks as m\n"
            "from powerinfer_b200 import synth\n"
            "for name in sorted(m.BASE):\n"
            "    for which in sorted(m.THRESHOLDS):\n"
            "        w = m.run_case(name, which)\n"
            "        assert w <= (5e-2 if m.BASE[name].wtype == synth.Q4_0 else 2e-2), (name, which, w)\n"
            "print('ok')\n")
    env = dict(os.environ, PI_FFN_FUSED="0")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
