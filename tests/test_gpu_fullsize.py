"""The sparse FFN operators at the headline configuration's full layer size (d 8192, F 28672, Q4_0 and FP16 rows), checked
through size-independent properties and against the CPU checker on a sample of rows (the full matrices would take the
checker minutes): exact zeros for inactive rows, gather == dense on active rows, exact homogeneity of the axpy under
scaling by two, a one-hot axpy against the dequantised row, run-to-run determinism."""
import numpy as np
import pytest

from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
D, F = 8192, 28672


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import ggml_ops
    return ggml_ops


@pytest.fixture(scope="module")
def oracle():
    from oracle import pio
    return pio.Oracle()


def device_weight(ops, wtype, gen):
    w = (torch.randn(F, D, device="cuda", generator=gen) * 0.02).to(torch.float16)
    if wtype == synth.F16:
        return ops.Weight(wtype, w.view(torch.uint8).reshape(-1), F, D), None
    raw = ops.quantize_q4_0(w.float())                                     # ggml block bytes, then the planar upload layout
    dev = torch.empty_like(raw)
    from powerinfer_b200._lib import check, lib
    check(lib.pi_q4_0_repack(raw.data_ptr(), dev.data_ptr(), F, D, torch.cuda.current_stream().cuda_stream))
    return ops.Weight(wtype, dev, F, D), raw.reshape(F, D // 32 * 18)


@pytest.mark.parametrize("wtype", [synth.Q4_0, synth.F16])
@pytest.mark.parametrize("T", [1, 8])
def test_full_size_layer_properties(ops, oracle, wtype, T):
    gen = torch.Generator(device="cuda"); gen.manual_seed(1234 + wtype)
    rng = np.random.default_rng(5 + wtype + T)
    W, raw = device_weight(ops, wtype, gen)
    Wt, raw_t = device_weight(ops, wtype, gen)
    x = torch.randn(T, D, device="cuda", generator=gen)
    prof = synth.zipf_profile(F, 0.12)[rng.permutation(F)]
    mask = rng.random((T, F)) < prof[None, :]
    idx = torch.from_numpy(np.where(mask, 1.0, -1.0).astype(np.float32)).cuda()
    up = ops.ggml_mul_mat_idx(W, x, idx)
    assert torch.equal(up, ops.ggml_mul_mat_idx(W, x, idx))                # deterministic
    upc = up.cpu().numpy()
    assert not upc[~mask].any()                                            # inactive rows are exactly zero
    dense = ops.ggml_mul_mat(W, x).cpu().numpy()
    assert np.abs(upc[mask] - dense[mask]).max() <= 2e-4                   # gather == dense on the active rows
    # a sample of rows against the CPU checker (FP16-rounded / Q8_0-quantised activations, as the reference's CPU path)
    rows = np.sort(rng.choice(F, 48, replace=False))
    wt_host = (raw[rows].cpu().numpy() if wtype == synth.Q4_0 else W.data.view(torch.float16).reshape(F, D)[rows].cpu().numpy())
    ref = oracle.mul_mat(wtype, wt_host, len(rows), D, x.cpu().numpy())
    assert np.abs(dense[:, rows] - ref).max() <= 2e-4
    # axpy: scaling h by two scales every coefficient exactly (Q8_0 scale and FP16 rounding are both homogeneous in 2)
    # (0.5 is added to the active entries so that no block scale falls into the FP16 subnormals, where rounding is not)
    h = (torch.relu(up) + 0.5) * torch.from_numpy(mask).cuda()
    y1, y2 = ops.ggml_axpy(Wt, h, idx), ops.ggml_axpy(Wt, 2.0 * h, idx)
    assert torch.equal(y2, 2.0 * y1)
    assert torch.equal(y1, ops.ggml_axpy(Wt, h, idx))
    # one active neuron: the result is that row of down_t times its coefficient, one term, no summation order involved
    r = int(rows[7])
    h1 = torch.zeros(T, F, device="cuda"); h1[:, r] = 0.75
    idx1 = torch.full((T, F), -1.0, device="cuda"); idx1[:, r] = 1.0
    y = ops.ggml_axpy(Wt, h1, idx1).cpu().numpy()
    row = ops.dequantize(Wt)[r].cpu().numpy()
    coef = 0.75 if wtype == synth.F16 else float(np.float32(127) * np.float32(np.float16(np.float32(0.75) / np.float32(127.0))))
    # FP16 rows: one exact product.  Q4_0, one token: the nibble-to-float trick spends ~4 bits of the FP32 accumulator;
    # Q4_0 batches: weight and coefficient are each rounded to FP16 once
    rel = 1e-7 if wtype == synth.F16 else (4e-6 if T == 1 else 1e-3)
    assert np.abs(y - coef * row[None, :]).max() <= rel * np.abs(row).max()
