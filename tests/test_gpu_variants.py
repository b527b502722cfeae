"""Alternative launch sequences of the one-token step (diagnostic environment switches) must give the same results as the
default one: gather and axpy as two launches instead of the single-launch sparse FFN (PI_FFN_FUSED=0), the separate mask kernel instead of the activity masks written by the predictor's second mat-vec
(PI_FC2_MASKS=0, must agree bit for bit), that mat-vec through a kernel without the mask epilogue (PI_RING_W=0: the mask
kernel follows it), the list-driven sparse kernels instead of the mask-driven register-streaming ones (PI_ROWS=0), no
programmatic dependent launch (PI_PDL=0), the ring kernels with a block barrier per stage, the single-CTA norm.  Each
variant runs in a child process because the switches are read when an engine is created."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys, numpy as np
sys.path.insert(0, %r); sys.path.insert(0, %r + '/tests/golden')
import torch
import make_golden as mg
from powerinfer_b200 import synth, engine
out = {}
for name in ('llama_q4_0', 'llama_gqa_f16', 'falcon_f16', 'opt_f16'):
    spec = mg.MODEL_CASES[name]
    eng = engine.DecodeEngine(spec, synth.build_model(spec), max_batch=1)
    logs = []
    for pos, tok in enumerate([5, 17, 300, 41, 9, 77]):
        logs.append(eng.decode([tok], [pos])[0][0].copy())
    eng.status()
    eng.close()
    out[name] = np.stack(logs)
np.savez(sys.argv[1], **out)
""" % (ROOT, ROOT)


def run_variant(tmp_path, tag, env):
    import numpy as np
    path = str(tmp_path / f"{tag}.npz")
    e = dict(os.environ)
    e.update(env)
    subprocess.run([sys.executable, "-c", SCRIPT, path], check=True, env=e)
    return np.load(path)


def test_step_variants_agree(tmp_path):
    import numpy as np
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    base = run_variant(tmp_path, "base", {})
    for tag, env in (("two_kernel_ffn", {"PI_FFN_FUSED": "0"}), ("mask_kernel", {"PI_FC2_MASKS": "0"}), ("masks_by_follow_up_kernel", {"PI_RING_W": "0"}), ("list_kernels", {"PI_ROWS": "0"}), ("no_pdl", {"PI_PDL": "0"}), ("rw4", {"PI_RING_RW": "4"}),
                     ("block_barrier_ring", {"PI_RING_W": "0", "PI_RING_G": "0", "PI_ROWS": "0"}), ("single_cta_norm", {"PI_NORM_CLUSTER": "0"})):
        got = run_variant(tmp_path, tag, env)
        for name in base.files:
            err = float(np.abs(got[name] - base[name]).max())
            assert err <= 5e-3, (tag, name, err)      # same math, different summation order / activation re-rounding
