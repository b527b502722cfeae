"""Parity of the CUDA operators (through the C ABI) with the CPU checker and the reference's golden outputs.

Tolerances: quantisers and index lists bit-exact; mat-vec style results within 2e-4 absolute of the
reference (its outputs here are O(0.1-1); the stated bars are 2e-2 for FP16 and 5e-2 for Q4_0 logits),
the only difference being the order of FP32 additions.
"""
import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
ATOL = 2e-4


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from powerinfer_b200 import ggml_ops
    return ggml_ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_q4_0_quantiser_bit_exact(ops, oracle, golden_ops):
    xs = np.random.default_rng(7).standard_normal((3, 512), dtype=np.float32)
    q = ops.quantize_q4_0(dev(xs * np.float32(0.02))).cpu().numpy()
    assert np.array_equal(q, golden_ops["q4_0"])
    q8 = ops.quantize_q8_0(dev(xs)).cpu().numpy()
    assert np.array_equal(q8, golden_ops["q8_0"])
    # edge cases: all-zero block, ties in magnitude, huge and tiny values
    e = np.zeros((4, 256), np.float32)
    e[1, :32] = 1.0
    e[1, 5] = -1.0
    e[2] = np.random.default_rng(1).standard_normal(256).astype(np.float32) * 1e-30
    e[3] = np.random.default_rng(2).standard_normal(256).astype(np.float32) * 6e4
    assert np.array_equal(ops.quantize_q4_0(dev(e)).cpu().numpy(), oracle.quantize_q4_0(e))
    assert np.array_equal(ops.quantize_q8_0(dev(e)).cpu().numpy(), oracle.quantize_q8_0(e))


def test_q4_0_repack_round_trip(ops, oracle):
    w = (np.random.default_rng(3).standard_normal((64, 512)) * 0.02).astype(np.float32)
    q = synth.quantize_q4_0(w)
    W = ops.upload_weight(q, synth.Q4_0, 64, 512)
    deq = ops.dequantize(W).cpu().numpy()
    assert np.array_equal(deq.reshape(-1), oracle.dequantize_q4_0(q.reshape(-1), w.size))


@pytest.mark.parametrize("name", sorted(mg.op_cases()))
def test_sparse_ops_vs_reference_golden(ops, golden_ops, name):
    c = mg.op_cases()[name]
    x, W, Wt, idx = mg.op_inputs(c)
    Wd = ops.upload_weight(W, c["wtype"], c["F"], c["d"])
    Wtd = ops.upload_weight(Wt, c["wtype"], c["F"], c["d"])
    up = ops.ggml_mul_mat_idx(Wd, dev(x), dev(idx))
    ref_up = golden_ops[name + ".up"]
    assert np.abs(up.cpu().numpy() - ref_up).max() <= ATOL
    assert np.all(up.cpu().numpy()[idx < 0] == 0.0)                      # inactive rows are exactly zero
    h = np.maximum(ref_up, 0)
    down = ops.ggml_axpy(Wtd, dev(h), dev(idx)).cpu().numpy()
    assert np.abs(down - golden_ops[name + ".down"]).max() <= ATOL
    down2 = ops.ggml_axpy(Wtd, dev(h), dev(idx)).cpu().numpy()
    assert np.array_equal(down, down2)                                  # fixed summation order
    dense = ops.ggml_mul_mat(Wd, dev(x)).cpu().numpy()
    assert np.abs(dense - golden_ops[name + ".dense"]).max() <= ATOL


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
@pytest.mark.parametrize("T", [1, 3, 8, 16])
def test_sparse_ops_vs_oracle_batches_and_buckets(ops, oracle, wtype, T):
    """Union list across the batch with a per-token predicate, and the gpu_bucket (row subset) form."""
    rng = np.random.default_rng(100 * wtype + T)
    d, F = 512, 2048
    x = rng.standard_normal((T, d), dtype=np.float32)
    Wf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    Wtf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    W = synth.quantize_q4_0(Wf) if wtype == synth.Q4_0 else Wf.astype(np.float16)
    Wt = synth.quantize_q4_0(Wtf) if wtype == synth.Q4_0 else Wtf.astype(np.float16)
    idx = (rng.random((T, F)) - 0.85).astype(np.float32)
    ref_up = oracle.mul_mat_idx(wtype, W, F, d, x, idx)
    h = np.maximum(ref_up, 0)
    ref_down = oracle.axpy(wtype, Wt, F, d, h, idx, np.zeros(F, np.int32))
    Wd, Wtd = ops.upload_weight(W, wtype, F, d), ops.upload_weight(Wt, wtype, F, d)
    up = ops.ggml_mul_mat_idx(Wd, dev(x), dev(idx)).cpu().numpy()
    assert np.abs(up - ref_up).max() <= ATOL
    down = ops.ggml_axpy(Wtd, dev(h), dev(idx)).cpu().numpy()
    assert np.abs(down - ref_down).max() <= ATOL
    # bucket: this device holds whole 32-neuron blocks 0, 2, 4, ...; the CPU op sees the complement as gpu_idx == 1
    blocks = np.arange(0, F // 32, 2)
    bucket = (blocks[:, None] * 32 + np.arange(32)[None, :]).reshape(-1).astype(np.int32)
    rb = W.shape[1] if wtype == synth.Q4_0 else None
    Wb = W[bucket]
    Wtb = Wt[bucket]
    Wbd, Wtbd = ops.upload_weight(Wb, wtype, len(bucket), d), ops.upload_weight(Wtb, wtype, len(bucket), d)
    gpu_idx = np.ones(F, np.int32)
    gpu_idx[bucket] = 0
    ref_up_b = oracle.mul_mat_idx(wtype, W, F, d, x, idx, gpu_idx)
    up_b = ops.ggml_mul_mat_idx(Wbd, dev(x), dev(idx), dev(bucket), result_ne0=F).cpu().numpy()
    assert np.abs(up_b - ref_up_b).max() <= ATOL
    ref_down_b = oracle.axpy(wtype, Wt, F, d, h, idx, gpu_idx)
    down_b = ops.ggml_axpy(Wtbd, dev(h), dev(idx), dev(bucket)).cpu().numpy()
    assert np.abs(down_b - ref_down_b).max() <= ATOL


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
@pytest.mark.parametrize("T", [1, 4, 16])
@pytest.mark.parametrize("gated", [True, False])
def test_sparse_ffn_one_call_vs_oracle_nodes(ops, oracle, wtype, T, gated):
    """pi_sparse_ffn against the reference's node sequence on the CPU: mul_mat_idx (up, gate), relu / mul (or bias add +
    relu), axpy; full and bucketed (hot rows only) forms."""
    rng = np.random.default_rng(7 + 10 * wtype + T + (100 if gated else 0))
    d, F = 512, 2048
    x = rng.standard_normal((T, d), dtype=np.float32)
    mats = [rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.05) for _ in range(3)]
    q = [synth.quantize_q4_0(m) if wtype == synth.Q4_0 else m.astype(np.float16) for m in mats]
    bias = None if gated else (rng.standard_normal(F).astype(np.float32) * np.float32(0.1))
    idx = (rng.random((T, F)) - 0.8).astype(np.float32)
    zeros = np.zeros(F, np.int32)

    def ref_ffn(gpu_idx):
        up = oracle.mul_mat_idx(wtype, q[0], F, d, x, idx, gpu_idx)
        if gated:
            gate = oracle.mul_mat_idx(wtype, q[1], F, d, x, idx, gpu_idx)
            h = np.maximum(gate, 0) * up
        else:
            h = np.maximum(up + bias[None, :], 0)                       # the bias add is dense, as the graph's ggml_add
        return oracle.axpy(wtype, q[2], F, d, h, idx, gpu_idx)

    W = [ops.upload_weight(m, wtype, F, d) for m in q]
    got = ops.sparse_ffn(W[0], W[1] if gated else None, W[2], dev(x), dev(idx), up_bias=dev(bias) if bias is not None else None)
    ref = ref_ffn(zeros)
    assert np.abs(got.cpu().numpy() - ref).max() <= 5 * ATOL, np.abs(got.cpu().numpy() - ref).max()
    again = ops.sparse_ffn(W[0], W[1] if gated else None, W[2], dev(x), dev(idx), up_bias=dev(bias) if bias is not None else None)
    assert torch.equal(got, again)
    # hot rows only (whole 32-neuron blocks 1, 3, 5, ...)
    blocks = np.arange(1, F // 32, 2)
    bucket = (blocks[:, None] * 32 + np.arange(32)[None, :]).reshape(-1).astype(np.int32)
    gpu_idx = np.ones(F, np.int32)
    gpu_idx[bucket] = 0
    Wb = [ops.upload_weight(m[bucket], wtype, len(bucket), d) for m in q]
    got_b = ops.sparse_ffn(Wb[0], Wb[1] if gated else None, Wb[2], dev(x), dev(idx), gpu_bucket=dev(bucket),
                           up_bias=dev(bias) if bias is not None else None)
    ref_b = ref_ffn(gpu_idx)
    assert np.abs(got_b.cpu().numpy() - ref_b).max() <= 5 * ATOL, np.abs(got_b.cpu().numpy() - ref_b).max()
    assert ops.last_op_status() == 0                                  # no bounded wait of the batch kernels ran out


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_hot_rows_from_placement_match_the_cpu_split(ops, oracle, wtype):
    """The placement module's gpu_idx / gpu_bucket drive both halves of the reference's hybrid split: the device computes
    the hot rows (bucket form), the CPU operator the cold ones (gpu_idx form); their sum is the full result
    (llama.cpp:4581-4594)."""
    from powerinfer_b200 import placement
    rng = np.random.default_rng(3 + wtype)
    d, F, T = 512, 2048, 2
    prof = synth.zipf_profile(F, 0.15)[rng.permutation(F)]
    gpu_idx, bucket = placement.bucket_of_whole_blocks(prof, 768)
    x = rng.standard_normal((T, d), dtype=np.float32)
    mats = [rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.05) for _ in range(3)]
    q = [synth.quantize_q4_0(m) if wtype == synth.Q4_0 else m.astype(np.float16) for m in mats]
    idx = np.where(rng.random((T, F)) < prof[None, :], 1.0, -1.0).astype(np.float32)
    zeros = np.zeros(F, np.int32)

    def cpu_ffn(gi):
        up = oracle.mul_mat_idx(wtype, q[0], F, d, x, idx, gi)
        gate = oracle.mul_mat_idx(wtype, q[1], F, d, x, idx, gi)
        return oracle.axpy(wtype, q[2], F, d, np.maximum(gate, 0) * up, idx, gi)

    Wb = [ops.upload_weight(m[bucket], wtype, len(bucket), d) for m in q]
    hot = ops.sparse_ffn(Wb[0], Wb[1], Wb[2], dev(x), dev(idx), gpu_bucket=dev(bucket)).cpu().numpy()
    ref_hot = cpu_ffn(1 - gpu_idx)                                # the CPU op skips rows flagged 1: flag the cold ones -> hot part
    assert np.abs(hot - ref_hot).max() <= 5 * ATOL
    cold = cpu_ffn(gpu_idx)                                       # what the reference's CPU half computes
    full = cpu_ffn(zeros)
    assert np.abs((hot + cold) - full).max() <= 2e-3              # Q4_0 coefficients are per 32-neuron block: whole blocks keep them equal


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
@pytest.mark.parametrize("T", [2, 8, 13, 32])
def test_small_batch_tensor_core_kernels_vs_oracle(ops, oracle, wtype, T):
    """Shapes that take the tensor-core paths (2..32 tokens, 1024-column slices): ggml_mul_mat_idx (FP16 rows), ggml_axpy
    (FP16 and Q4_0 rows) and the one-call FFN against the CPU operators, full and bucketed.  The Q4_0 axpy rounds the
    dequantised weight and the coefficient to FP16 once each (the CPU multiplies (q-8)*b8 as integers): 1e-3 there."""
    rng = np.random.default_rng(900 + T + wtype)
    d, F = 2048, 1536
    q4 = wtype == synth.Q4_0
    atol_axpy = 1e-3 if q4 else ATOL
    x = rng.standard_normal((T, d), dtype=np.float32)
    mk = lambda: rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    W, Wg, Wt = ((synth.quantize_q4_0(m) if q4 else m.astype(np.float16)) for m in (mk(), mk(), mk()))
    idx = (rng.random((T, F)) - 0.8).astype(np.float32)
    zeros = np.zeros(F, np.int32)
    Wd, Wgd, Wtd = (ops.upload_weight(m, wtype, F, d) for m in (W, Wg, Wt))
    ref_up = oracle.mul_mat_idx(wtype, W, F, d, x, idx, zeros)
    up = ops.ggml_mul_mat_idx(Wd, dev(x), dev(idx)).cpu().numpy()
    assert np.abs(up - ref_up).max() <= ATOL
    h = np.maximum(ref_up, 0)
    ref_down = oracle.axpy(wtype, Wt, F, d, h, idx, zeros)
    down = ops.ggml_axpy(Wtd, dev(h), dev(idx)).cpu().numpy()
    assert np.abs(down - ref_down).max() <= atol_axpy, np.abs(down - ref_down).max()
    assert np.array_equal(down, ops.ggml_axpy(Wtd, dev(h), dev(idx)).cpu().numpy())
    ref_gate = oracle.mul_mat_idx(wtype, Wg, F, d, x, idx, zeros)
    ref_ffn = oracle.axpy(wtype, Wt, F, d, np.maximum(ref_gate, 0) * ref_up, idx, zeros)
    ffn = ops.sparse_ffn(Wd, Wgd, Wtd, dev(x), dev(idx)).cpu().numpy()
    assert np.abs(ffn - ref_ffn).max() <= 5 * atol_axpy
    blocks = np.arange(0, F // 32, 3)
    bucket = (blocks[:, None] * 32 + np.arange(32)[None, :]).reshape(-1).astype(np.int32)
    gpu_idx = np.ones(F, np.int32)
    gpu_idx[bucket] = 0
    Wtb = ops.upload_weight(Wt[bucket], wtype, len(bucket), d)
    down_b = ops.ggml_axpy(Wtb, dev(h), dev(idx), dev(bucket)).cpu().numpy()
    assert np.abs(down_b - oracle.axpy(wtype, Wt, F, d, h, idx, gpu_idx)).max() <= atol_axpy


@pytest.mark.parametrize("T", [2, 5, 8, 11, 16])
@pytest.mark.parametrize("d", [256, 1024, 2560])
def test_q4_0_small_batch_integer_tensor_core_kernel_vs_oracle(ops, oracle, T, d):
    """Q4_0 rows with 2+ tokens take the integer tensor-core kernel (tiles of 16 or 8 row vectors, launches of 8 tokens): dense
    with a ragged last tile, ggml_mul_mat_idx over a ragged list, bucketed rows, and the gated pair inside the one-call
    FFN, against the CPU operators.  The integer block dots are exact; only the FP32 order over the blocks differs."""
    rng = np.random.default_rng(1300 + T + d)
    F = 2400 + 16 + 5                                             # >= 148 tiles of 16 rows, last tile ragged
    x = rng.standard_normal((T, d), dtype=np.float32)
    mk = lambda n: synth.quantize_q4_0(rng.standard_normal((n, d), dtype=np.float32) * np.float32(0.02))
    W, Wg = mk(F), mk(F)
    Wd, Wgd = ops.upload_weight(W, synth.Q4_0, F, d), ops.upload_weight(Wg, synth.Q4_0, F, d)
    ref = oracle.mul_mat(synth.Q4_0, W, F, d, x)
    out = ops.ggml_mul_mat(Wd, dev(x)).cpu().numpy()
    assert np.abs(out - ref).max() <= ATOL, np.abs(out - ref).max()
    idx = (rng.random((T, F)) - 0.7).astype(np.float32)
    zeros = np.zeros(F, np.int32)
    ref_up = oracle.mul_mat_idx(synth.Q4_0, W, F, d, x, idx, zeros)
    up = ops.ggml_mul_mat_idx(Wd, dev(x), dev(idx)).cpu().numpy()
    assert np.abs(up - ref_up).max() <= ATOL
    assert np.array_equal(up == 0, ref_up == 0) or np.abs(up - ref_up).max() <= ATOL
    bucket = np.sort(rng.choice(F, 333, replace=False)).astype(np.int32)
    gpu_idx = np.ones(F, np.int32)
    gpu_idx[bucket] = 0
    Wb = ops.upload_weight(W[bucket], synth.Q4_0, len(bucket), d)
    up_b = ops.ggml_mul_mat_idx(Wb, dev(x), dev(idx), dev(bucket), result_ne0=F).cpu().numpy()
    assert np.abs(up_b - oracle.mul_mat_idx(synth.Q4_0, W, F, d, x, idx, gpu_idx)).max() <= ATOL
    if d % 1024 == 0 or d == 256:
        Fd = F // 32 * 32
        Wt = mk(d)[:, :0]                                         # placeholder keeps the generator sequence simple
        Wt = synth.quantize_q4_0(rng.standard_normal((Fd, d), dtype=np.float32) * np.float32(0.02))
        Wtd = ops.upload_weight(Wt, synth.Q4_0, Fd, d)
        Wd2, Wgd2 = ops.upload_weight(W[:Fd], synth.Q4_0, Fd, d), ops.upload_weight(Wg[:Fd], synth.Q4_0, Fd, d)
        idx2 = np.ascontiguousarray(idx[:, :Fd])
        z2 = np.zeros(Fd, np.int32)
        r_up = oracle.mul_mat_idx(synth.Q4_0, W[:Fd], Fd, d, x, idx2, z2)
        r_gate = oracle.mul_mat_idx(synth.Q4_0, Wg[:Fd], Fd, d, x, idx2, z2)
        r_ffn = oracle.axpy(synth.Q4_0, Wt, Fd, d, np.maximum(r_gate, 0) * r_up, idx2, z2)
        ffn = ops.sparse_ffn(Wd2, Wgd2, Wtd, dev(x), dev(idx2)).cpu().numpy()
        assert np.abs(ffn - r_ffn).max() <= 5e-3, np.abs(ffn - r_ffn).max()


def test_predictor_and_active_list(ops, oracle):
    spec = synth.ModelSpec(n_layer=1, d=512, n_ff=4096, rank=128, firing=0.1, seed=5)
    t = synth.build_model(spec)
    rng = np.random.default_rng(0)
    for T in (1, 4):
        p = rng.standard_normal((T, spec.d), dtype=np.float32)
        hid = np.maximum(oracle.mul_mat(synth.F16, t["blk.0.fc1.weight"], spec.rank, spec.d, p), 0)
        ref = oracle.mul_mat(synth.F16, t["blk.0.fc2.weight"], spec.n_ff, spec.rank, hid)
        fc1 = ops.upload_weight(t["blk.0.fc1.weight"], synth.F16, spec.rank, spec.d)
        fc2 = ops.upload_weight(t["blk.0.fc2.weight"], synth.F16, spec.n_ff, spec.rank)
        idx = ops.predictor(fc1, fc2, dev(p))
        got = idx.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-4
        # index sets: bit-exact except neurons whose logit lies within 1e-3 of the threshold
        sure = np.abs(ref) > 1e-3
        assert np.array_equal((got >= 0)[sure], (ref >= 0)[sure])
        lst, cnt = ops.active_list(idx)
        n = int(cnt.item())
        want = np.nonzero((got >= 0).any(axis=0))[0]
        assert n == len(want) and np.array_equal(lst[:n].cpu().numpy(), want)


def test_active_list_edges(ops):
    for F in (32, 1000, 1280, 49152):
        for kind in ("empty", "full", "one", "ragged"):
            idx = -np.ones((1, F), np.float32)
            if kind == "full":
                idx[:] = 1
            elif kind == "one":
                idx[0, F - 1] = 0.0
            elif kind == "ragged":
                idx[0, ::7] = 0.5
            lst, cnt = ops.active_list(dev(idx))
            want = np.nonzero(idx[0] >= 0)[0]
            assert int(cnt.item()) == len(want)
            assert np.array_equal(lst[:len(want)].cpu().numpy(), want)


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
@pytest.mark.parametrize("T", [1, 5])
def test_sparse_ops_edge_masks_and_threshold(ops, oracle, wtype, T):
    """No neuron active, every neuron active, logits exactly at a non-zero threshold, NaN logits (active: the reference
    skips a row when `logit < threshold`, which is false for NaN) and bad arguments rejected before any launch."""
    rng = np.random.default_rng(40 + wtype + T)
    d, F = 512, 1024
    x = rng.standard_normal((T, d), dtype=np.float32)
    mats = [rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.03) for _ in range(2)]
    q = [synth.quantize_q4_0(m) if wtype == synth.Q4_0 else m.astype(np.float16) for m in mats]
    W, Wt = (ops.upload_weight(m, wtype, F, d) for m in q)
    zeros = np.zeros(F, np.int32)
    base = rng.standard_normal((T, F)).astype(np.float32)
    cases = {"none": np.full((T, F), -1.0, np.float32), "all": np.full((T, F), 2.0, np.float32)}
    at = base.copy(); at[:, ::3] = 0.25                                   # exactly at the threshold: active (>=)
    cases["at_threshold"] = at
    nan = base.copy(); nan[:, ::5] = np.nan
    cases["nan"] = nan
    saved = ops.sparse_pred_threshold
    try:
        for name, idx in cases.items():
            thr = 0.25 if name == "at_threshold" else 0.0
            ops.sparse_pred_threshold = thr
            ref_up = oracle.mul_mat_idx(wtype, q[0], F, d, x, idx, zeros, thr)
            up = ops.ggml_mul_mat_idx(W, dev(x), dev(idx)).cpu().numpy()
            assert np.abs(up - ref_up).max() <= ATOL, name
            h = np.maximum(ref_up, 0)
            ref_down = oracle.axpy(wtype, q[1], F, d, h, idx, zeros, thr)
            down = ops.ggml_axpy(Wt, dev(h), dev(idx)).cpu().numpy()
            assert np.abs(down - ref_down).max() <= ATOL, name
            if name == "none":
                assert not up.any() and not down.any()
            if name == "nan":
                assert up[:, ::5].any()                                   # computed, as on the CPU
    finally:
        ops.sparse_pred_threshold = saved
    from powerinfer_b200 import _lib
    xd, id_ = dev(x), dev(cases["all"])
    out = torch.empty(T, F, dtype=torch.float32, device="cuda")
    ws = torch.empty(1 << 22, dtype=torch.uint8, device="cuda")
    # fewer destination rows than weight rows: rejected with a message, nothing launched
    rc = _lib.lib.pi_mul_mat_idx(wtype, W.ptr, F, d, xd.data_ptr(), T, id_.data_ptr(), F, None, 0.0, out.data_ptr(), F - 32,
                                 ws.data_ptr(), ws.numel(), None)
    assert rc == 1 and b"n_w_rows" in _lib.lib.pi_last_error()
    rc = _lib.lib.pi_mul_mat_idx(wtype, W.ptr, F, d, xd.data_ptr(), T, id_.data_ptr(), F, None, 0.0, out.data_ptr(), F,
                                 ws.data_ptr(), 1024, None)
    assert rc != 0 and b"workspace" in _lib.lib.pi_last_error()           # too small a workspace is an error, not a fault


def test_norms_rope_bit_exact(ops, golden_ops):
    xs = np.random.default_rng(7).standard_normal((3, 512), dtype=np.float32)
    assert np.array_equal(ops.ggml_rms_norm(dev(xs), 1e-5).cpu().numpy(), golden_ops["rms_norm"])
    got = ops.ggml_norm(dev(xs), 1e-5).cpu().numpy()
    assert np.abs(got - golden_ops["norm"]).max() <= 1e-6
    tab = ops.rope_table(320, 128, 10000.0)
    tab64 = ops.rope_table(320, 64, 10000.0)
    for pos in (0, 1, 37, 300):
        p = torch.tensor([pos], dtype=torch.int32, device="cuda")
        y = ops.ggml_rope_custom(dev(xs[0].reshape(1, 4, 128)), p, 128, 0, tab).cpu().numpy().reshape(4, 128)
        assert np.array_equal(y, golden_ops[f"rope_{pos}"])
        y = ops.ggml_rope_custom(dev(xs[0].reshape(1, 8, 64)), p, 64, 2, tab64).cpu().numpy().reshape(8, 64)
        assert np.array_equal(y, golden_ops[f"rope_neox_{pos}"])


def test_norm_weight_bias_and_wide_rows(ops, oracle):
    rng = np.random.default_rng(9)
    for n in (256, 4096, 8192, 12288):
        x = rng.standard_normal((2, n), dtype=np.float32)
        w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        b = (0.1 * rng.standard_normal(n)).astype(np.float32)
        ref = oracle.rms_norm(x, 1e-5) * w
        assert np.abs(ops.ggml_rms_norm(dev(x), 1e-5, dev(w)).cpu().numpy() - ref).max() <= 1e-6
        ref = oracle.norm(x, 1e-5) * w + b
        assert np.abs(ops.ggml_norm(dev(x), 1e-5, dev(w), dev(b)).cpu().numpy() - ref).max() <= 2e-6


@pytest.mark.parametrize("n_head,n_head_kv,hd", [(4, 4, 64), (8, 2, 128), (8, 8, 32)])
def test_attention_decode_vs_oracle(ops, oracle, n_head, n_head_kv, hd):
    """Feed 40 positions one by one; compare with the CPU restatement of llm_build_kqv (same FP16 roundings)."""
    rng = np.random.default_rng(n_head * 100 + hd)
    n_ctx, dkv, d = 64, n_head_kv * hd, n_head * hd
    kc = torch.zeros(1, n_ctx, dkv, dtype=torch.float16, device="cuda")
    vc = torch.zeros(1, n_ctx, dkv, dtype=torch.float16, device="cuda")
    K = np.zeros((n_ctx, dkv), np.float16)
    V = np.zeros((n_ctx, dkv), np.float16)
    group = n_head // n_head_kv
    for pos in range(40):
        q = rng.standard_normal((1, d), dtype=np.float32)
        k = rng.standard_normal((1, dkv), dtype=np.float32)
        v = rng.standard_normal((1, dkv), dtype=np.float32)
        out = ops.attention_decode(dev(q), dev(k), dev(v), kc, vc, torch.tensor([pos], dtype=torch.int32, device="cuda"),
                                   n_head, n_head_kv).cpu().numpy()[0]
        K[pos], V[pos] = k[0].astype(np.float16), v[0].astype(np.float16)
        ref = np.zeros(d, np.float32)
        scale = np.float32(1.0) / np.sqrt(np.float32(hd))
        for h in range(n_head):
            hk = h // group
            q16 = q[0, h * hd:(h + 1) * hd].astype(np.float16).astype(np.float32)
            s = (K[:pos + 1, hk * hd:(hk + 1) * hd].astype(np.float32) @ q16) * scale
            p = oracle.soft_max(s.astype(np.float32)[None, :])[0].astype(np.float16).astype(np.float32)
            ref[h * hd:(h + 1) * hd] = p @ V[:pos + 1, hk * hd:(hk + 1) * hd].astype(np.float32)
        assert np.abs(out - ref).max() <= 2e-3, pos
    assert np.array_equal(kc[0].cpu().numpy()[:40], K[:40])
