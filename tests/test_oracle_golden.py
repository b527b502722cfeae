"""The CPU checker (oracle/pi_oracle.c) against fixtures produced by the reference's own CPU code.

tests/golden/*.npz were written by tests/golden/make_golden.py from oracle/_ref (the reference's ggml.c and
llama.cpp compiled unmodified, one thread).  The restatement follows the reference's AVX2 lane order, so
the comparison is bit-exact, not a tolerance.
"""
import os

import numpy as np
import pytest

import make_golden as mg
from oracle import pio
from powerinfer_b200 import synth

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(mg.op_cases()))
def test_sparse_ops_bit_exact(oracle, golden_ops, name):
    c = mg.op_cases()[name]
    x, W, Wt, idx = mg.op_inputs(c)
    up = oracle.mul_mat_idx(c["wtype"], W, c["F"], c["d"], x, idx)
    assert np.array_equal(up, golden_ops[name + ".up"])
    h = np.maximum(up, 0)
    down = oracle.axpy(c["wtype"], Wt, c["F"], c["d"], h, idx, np.zeros(c["F"], np.int32))
    assert np.array_equal(down, golden_ops[name + ".down"])
    assert np.array_equal(oracle.mul_mat(c["wtype"], W, c["F"], c["d"], x), golden_ops[name + ".dense"])
    # inactive rows are exactly zero, active ones are the dense product
    act = idx >= 0.0
    assert np.all(up[~act] == 0.0)
    assert np.array_equal(up[act], golden_ops[name + ".dense"][act])


def test_small_nodes_bit_exact(oracle, golden_ops):
    xs = np.random.default_rng(7).standard_normal((3, 512), dtype=np.float32)
    assert np.array_equal(oracle.rms_norm(xs, 1e-5), golden_ops["rms_norm"])
    assert np.array_equal(oracle.norm(xs, 1e-5), golden_ops["norm"])
    sm = xs.copy()
    sm[:, 400:] = -np.inf
    assert np.array_equal(oracle.soft_max(sm), golden_ops["soft_max"])
    for pos in (0, 1, 37, 300):
        assert np.array_equal(oracle.rope(xs[0], 128, 4, pos, 10000.0, False), golden_ops[f"rope_{pos}"])
        assert np.array_equal(oracle.rope(xs[0], 64, 8, pos, 10000.0, True), golden_ops[f"rope_neox_{pos}"])
    assert np.array_equal(oracle.quantize_q8_0(xs), golden_ops["q8_0"])
    assert np.array_equal(oracle.quantize_q4_0(xs * 0.02), golden_ops["q4_0"])
    assert np.array_equal(synth.quantize_q4_0(xs * np.float32(0.02)).reshape(-1), golden_ops["q4_0"])


def test_gpu_idx_rows_are_skipped(oracle):
    """gpu_idx[r] == 1 marks a row that lives elsewhere: the CPU op writes 0 / skips it (ggml.c:14256, 14424)."""
    c = dict(wtype=synth.F16, d=256, F=1280, T=1, kind="full", seed=5)
    x, W, Wt, idx = mg.op_inputs(c)
    gi = np.zeros(1280, np.int32)
    gi[::3] = 1
    up = oracle.mul_mat_idx(synth.F16, W, 1280, 256, x, idx, gi)
    assert np.all(up[0, ::3] == 0) and np.all(up[0, 1::3] != 0)
    full = oracle.axpy(synth.F16, Wt, 1280, 256, np.abs(up) + 1, idx, np.zeros(1280, np.int32))
    part = oracle.axpy(synth.F16, Wt, 1280, 256, np.abs(up) + 1, idx, gi)
    rest = oracle.axpy(synth.F16, Wt, 1280, 256, np.abs(up) + 1, idx, 1 - gi)
    assert np.allclose(part + rest, full, atol=1e-5)


@pytest.mark.parametrize("name", sorted(mg.MODEL_CASES))
def test_decode_matches_reference_llama_cpp(name):
    """Logits bit-exact and greedy stream identical to the reference's llama.cpp (CPU, 1 thread)."""
    spec = mg.MODEL_CASES[name]
    g = np.load(os.path.join(GOLD, f"model_{name}.npz"))
    assert bool(g["single_equals_batch"])          # the reference itself: batched prompt == token by token
    t = synth.build_model(spec)
    if synth.digest(t) != str(g["digest"]):
        pytest.fail("numpy's generator no longer reproduces the weights this fixture was made from; "
                    "regenerate with tests/golden/make_golden.py")
    om = pio.OracleModel(spec, t)
    toks = [int(v) for v in g["prompt"]]
    pos = 0
    for tk in toks[:-1]:
        om.decode(tk, pos)
        pos += 1
    cur = toks[-1]
    for s in range(mg.N_STEPS):
        lg = om.decode(cur, pos)
        pos += 1
        assert np.array_equal(lg, g["logits"][s]), f"step {s}"
        cur = int(lg.argmax())
        assert cur == int(g["greedy"][s])
    om.close()


def test_firing_profile_is_zipf_with_requested_mean():
    p = synth.zipf_profile(11008, 0.10)
    assert abs(p.mean() - 0.10) < 1e-3 and p.max() <= 0.98 and np.all(np.diff(p) <= 1e-12)
    spec = synth.ModelSpec(n_layer=1, d=512, n_ff=4096, rank=128, firing=0.12, seed=3)
    t = synth.build_model(spec)
    om = pio.OracleModel(spec, t)
    rates = []
    for pos, tok in enumerate(np.random.default_rng(0).integers(0, spec.n_vocab, 12)):
        _, pred = om.decode(int(tok), pos, want_pred=True)
        rates.append((pred >= 0).mean())
    assert 0.06 < np.mean(rates) < 0.2, rates
