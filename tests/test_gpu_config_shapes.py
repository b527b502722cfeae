"""Operator parity at the per-layer shapes of every benchmarked configuration (the kernels pick their tile, slice and
ring geometry from the shape, so each shape is its own case):

    7B-shape        d  4096, F 11008, gated          13B microbench  d  5120, F 13824, gated, masks at 50/80/90/95 %
    falcon-40B      d  8192, F 32768, no gate        70B-shape       d  8192, F 28672, gated
    opt-175B        d 12288, F 49152, bias + relu

ggml_mul_mat_idx is held against the CPU checker on a sample of rows (plus: inactive rows exactly zero); ggml_axpy is held
against the CPU checker's axpy over the WHOLE matrix (every active row enters every output column, so nothing can hide).
Weights are made on the device and copied back for the checker.  The 2e-4 bar of the other operator tests is taken
relative to the largest reference value (outputs here reach 10 and more, and the FP32 sums run over thousands of rows);
the stated bars are 2e-2 (FP16) and 5e-2 (Q4_0) on logits."""
import ctypes as C

import numpy as np
import pytest

from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
RTOL = 2e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import ggml_ops
    return ggml_ops


def device_weight(ops, wtype, F, D, gen):
    """A random weight matrix on the device in upload layout + the host copy in the checker's (ggml) layout."""
    from powerinfer_b200._lib import check, lib
    w = (torch.randn(F, D, device="cuda", generator=gen) * 0.02).to(torch.float16)
    if wtype == synth.F16:
        return ops.Weight(wtype, w.view(torch.uint8).reshape(-1), F, D), w.cpu().numpy()
    raw = ops.quantize_q4_0(w.float())
    del w
    dev = torch.empty_like(raw)
    check(lib.pi_q4_0_repack(raw.data_ptr(), dev.data_ptr(), F, D, torch.cuda.current_stream().cuda_stream))
    return ops.Weight(wtype, dev, F, D), raw.reshape(F, D // 32 * 18).cpu().numpy()


def zipf_masks(rng, F, T, density):
    prof = synth.zipf_profile(F, density)[rng.permutation(F)]
    return rng.random((T, F)) < prof[None, :]


def check_layer(ops, oracle, wtype, D, F, gated, bias, cases, seed):
    gen = torch.Generator(device="cuda"); gen.manual_seed(seed)
    rng = np.random.default_rng(seed)
    up, up_h = device_weight(ops, wtype, F, D, gen)
    gate, gate_h = device_weight(ops, wtype, F, D, gen) if gated else (None, None)
    down, down_h = device_weight(ops, wtype, F, D, gen)
    up_b = (rng.standard_normal(F).astype(np.float32) * 0.1) if bias else None
    up_bd = torch.from_numpy(up_b).cuda() if bias else None
    for T, density in cases:
        x = torch.randn(T, D, device="cuda", generator=gen)
        mask = zipf_masks(rng, F, T, density)
        idx_h = np.where(mask, 1.0, -1.0).astype(np.float32)
        idx = torch.from_numpy(idx_h).cuda()
        tag = f"T={T} density={density}"
        # ---- ggml_mul_mat_idx (up, and gate): zeros where inactive, sampled rows against the checker
        u = ops.ggml_mul_mat_idx(up, x, idx).cpu().numpy()
        assert not u[~mask].any(), tag
        rows = np.sort(rng.choice(F, 64, replace=False))
        xh = x.cpu().numpy()
        ref_u = oracle.mul_mat(wtype, np.ascontiguousarray(up_h[rows]), len(rows), D, xh) * mask[:, rows]
        assert np.abs(u[:, rows] - ref_u).max() <= RTOL * max(1.0, np.abs(ref_u).max()), tag
        if gated:
            g = ops.ggml_mul_mat_idx(gate, x, idx).cpu().numpy()
            ref_g = oracle.mul_mat(wtype, np.ascontiguousarray(gate_h[rows]), len(rows), D, xh) * mask[:, rows]
            assert np.abs(g[:, rows] - ref_g).max() <= RTOL * max(1.0, np.abs(ref_g).max()), tag
            h = np.maximum(g, 0.0) * u
        else:
            h = np.maximum(u + (up_b[None, :] if bias else 0.0), 0.0)
        h = np.ascontiguousarray(h, np.float32)
        # ---- ggml_axpy over the whole matrix
        ref_y = oracle.axpy(wtype, down_h, F, D, h, idx_h, np.zeros(F, np.int32))
        y = ops.ggml_axpy(down, torch.from_numpy(h).cuda(), idx).cpu().numpy()
        bar = RTOL * max(1.0, np.abs(ref_y).max())
        # Q4_0 batches round weight and coefficient to FP16 once each on the tensor-core path (<= 5e-4 per term)
        if wtype == synth.Q4_0 and T > 1:
            bar *= 5
        assert np.abs(y - ref_y).max() <= bar, (tag, float(np.abs(y - ref_y).max()), bar)
        # ---- the whole FFN as one call must agree with the node-by-node result
        f = ops.sparse_ffn(up, gate, down, x, idx, up_bias=up_bd).cpu().numpy()
        assert np.abs(f - ref_y).max() <= 2 * bar, (tag, "sparse_ffn", float(np.abs(f - ref_y).max()))


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_7b_layer_shape(ops, oracle, wtype):
    check_layer(ops, oracle, wtype, 4096, 11008, True, False, [(1, 0.10), (8, 0.10)], 101 + wtype)


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_13b_microbench_shape_all_sparsities_and_batches(ops, oracle, wtype):
    cases = [(T, dens) for dens in (0.50, 0.20, 0.10, 0.05) for T in (1, 4, 8, 16)]
    check_layer(ops, oracle, wtype, 5120, 13824, True, False, cases, 202 + wtype)


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_falcon_40b_layer_shape(ops, oracle, wtype):
    check_layer(ops, oracle, wtype, 8192, 32768, False, False, [(1, 0.10), (8, 0.10)], 303 + wtype)


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_70b_layer_shape(ops, oracle, wtype):
    check_layer(ops, oracle, wtype, 8192, 28672, True, False, [(1, 0.12), (8, 0.12)], 404 + wtype)


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_opt_175b_layer_shape(ops, oracle, wtype):
    check_layer(ops, oracle, wtype, 12288, 49152, False, True, [(1, 0.08), (8, 0.08)], 505 + wtype)


def test_q4_0_axpy_rows_longer_than_8192_columns(ops, oracle):
    """Q4_0 rows of 12288 columns at a small neuron count through all three axpy entry points."""
    from powerinfer_b200._lib import lib
    D, F = 12288, 2048
    gen = torch.Generator(device="cuda"); gen.manual_seed(77)
    rng = np.random.default_rng(77)
    down, down_h = device_weight(ops, synth.Q4_0, F, D, gen)
    up, _ = device_weight(ops, synth.Q4_0, F, D, gen)
    for T in (1, 3):
        mask = rng.random((T, F)) < 0.3
        idx_h = np.where(mask, 1.0, -1.0).astype(np.float32)
        h = (np.abs(rng.standard_normal((T, F))).astype(np.float32) + 0.1) * mask
        ref = oracle.axpy(synth.Q4_0, down_h, F, D, h, idx_h, np.zeros(F, np.int32))
        bar = RTOL * max(1.0, np.abs(ref).max()) * (5 if T > 1 else 1)
        hd, idxd = torch.from_numpy(h).cuda(), torch.from_numpy(idx_h).cuda()
        y = ops.ggml_axpy(down, hd, idxd).cpu().numpy()
        assert np.abs(y - ref).max() <= bar, (T, float(np.abs(y - ref).max()))
        if T == 1:
            got = torch.full((1, D), float("nan"), dtype=torch.float32, device="cuda")
            rc = lib.pi_axpy_static(synth.Q4_0, down.ptr, F, D, hd.data_ptr(), F, idxd.data_ptr(), F, None, C.c_float(0.0),
                                    got.data_ptr(), torch.cuda.current_stream().cuda_stream)
            assert rc == 0, lib.pi_last_error().decode()
            assert np.abs(got.cpu().numpy() - ref).max() <= bar
    # and the whole FFN as one call (no gate: h = relu(up . x)), checked through its own nodes
    x = torch.randn(1, D, device="cuda", generator=gen)
    mask = rng.random((1, F)) < 0.3
    idx_h = np.where(mask, 1.0, -1.0).astype(np.float32)
    idxd = torch.from_numpy(idx_h).cuda()
    u = ops.ggml_mul_mat_idx(up, x, idxd)
    hh = torch.relu(u)
    ref = oracle.axpy(synth.Q4_0, down_h, F, D, hh.cpu().numpy(), idx_h, np.zeros(F, np.int32))
    f = ops.sparse_ffn(up, None, down, x, idxd).cpu().numpy()
    assert np.abs(f - ref).max() <= RTOL * max(1.0, np.abs(ref).max())
