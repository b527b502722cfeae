"""pi_axpy_static: the axpy operator for callers that may not allocate device memory.

A host that owns every byte of HBM (a serving process with a fixed arena) can forbid a plug-in to call cudaMalloc, and
code that runs during a stream capture cannot allocate either; such callers have no workspace to hand to pi_axpy.  This
entry point takes its scratch from an array inside the library instead.  The test calls it through the C ABI twice in a
row with different masks (so stale scratch contents from the first call would show in the second) and compares with
pi_axpy given an ordinary workspace (both run the same kernels in the same order, so the outputs must be identical) and
with the CPU checker's axpy on the same inputs, within the 2e-4 tolerance the other operator tests use.  The file name
sorts last so that a run that stops at the first failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ATOL = 2e-4


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_axpy_static_matches_axpy_on_two_calls_in_a_row(wtype, oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import ggml_ops
    from powerinfer_b200._lib import lib
    rng = np.random.default_rng(42 + wtype)
    d, F = 1024, 4096
    Wf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    Wt = synth.quantize_q4_0(Wf) if wtype == synth.Q4_0 else Wf.astype(np.float16)
    Wd = ggml_ops.upload_weight(Wt, wtype, F, d)
    stream = torch.cuda.current_stream().cuda_stream
    for call, density in enumerate((0.30, 0.05)):
        idx = (rng.random((1, F)) - (1 - density)).astype(np.float32)          # a different mask on the second call
        h = np.abs(rng.standard_normal((1, F), dtype=np.float32)) * (idx >= 0)
        hd, idxd = dev(h), dev(idx)
        want = ggml_ops.ggml_axpy(Wd, hd, idxd)
        got = torch.full((1, d), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.pi_axpy_static(wtype, Wd.ptr, F, d, hd.data_ptr(), F, idxd.data_ptr(), F, None, C.c_float(0.0),
                                got.data_ptr(), stream)
        assert rc == 0, lib.pi_last_error().decode()
        torch.cuda.synchronize()
        assert np.abs(got.cpu().numpy() - want.cpu().numpy()).max() <= ATOL, f"call {call}"
        assert torch.equal(got, want), f"call {call}: same kernels, same order"
        ref = oracle.axpy(wtype, Wt, F, d, h, idx, np.zeros(F, np.int32))
        assert np.abs(got.cpu().numpy() - ref).max() <= ATOL, f"call {call}: against the CPU checker"
        assert lib.pi_op_status(None, stream) == 0, lib.pi_last_error().decode()     # the built-in array's status word: no wait ran out
        assert ggml_ops.last_op_status() == 0


def test_axpy_static_rejects_shapes_beyond_its_scratch():
    from powerinfer_b200._lib import lib
    assert lib.pi_axpy_static_max_bytes() == 24 << 20
    # validation comes before any CUDA call, so dummy pointers are never dereferenced
    rc = lib.pi_axpy_static(synth.F16, 256, 70000, 1024, 256, 70000, 256, 70000, None, C.c_float(0.0), 256, None)
    assert rc == 1 and b"pi_axpy" in lib.pi_last_error()
    rc = lib.pi_axpy_static(synth.F16, 256, 4096, 32768, 256, 4096, 256, 4096, None, C.c_float(0.0), 256, None)
    assert rc == 1 and b"16384" in lib.pi_last_error()
