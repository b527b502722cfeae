"""Generate the golden fixtures in this folder from the REFERENCE's own CPU code.

Run where the reference checkout is present (it is not needed afterwards):

    make -C oracle && python tests/golden/make_golden.py

ops.npz      outputs of the reference's ggml CPU ops (oracle/_ref/libpi_ref.so, one thread) on
             seeded inputs that tests regenerate from `op_cases()`.
model_*.npz  raw logits and greedy token ids of the reference's llama.cpp decode loop
             (oracle/_ref/ref_decode, one thread) on seeded synthetic PowerInfer GGUF models that tests
             regenerate from `MODEL_CASES`; the weights' SHA-256 is stored to detect RNG drift.

One thread is mandatory: with more, the reference's CPU axpy loses updates (ggml.c:14433-14458).
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from powerinfer_b200 import synth  # noqa: E402

N_PROMPT, N_STEPS = 8, 32

MODEL_CASES = {
    "llama_f16": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, seed=11),
    "llama_q4_0": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.Q4_0, seed=12),
    "llama_gqa_f16": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, n_head=8, n_head_kv=2, d=512, n_ff=1536,
                                     rank=96, seed=13, firing=0.2),
    "falcon_f16": synth.ModelSpec(arch=synth.ARCH_FALCON, wtype=synth.F16, n_head=8, n_head_kv=2, d=512, n_ff=2048,
                                  seed=14),
    "opt_f16": synth.ModelSpec(arch=synth.ARCH_OPT, wtype=synth.F16, seed=15, norm_eps=0.0),
    "bamboo_f16": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, gate_sym=True, seed=16),
}


# Two-layer models at the PER-LAYER SHAPES of the benchmarked configurations (vocabulary cut to 1024 rows to keep the
# fixtures small): the kernels choose tile, slice and ring geometry from the layer shape, so parity on toy shapes does not
# cover them.  `python make_golden.py shapes` regenerates these (minutes of CPU time and ~10 GB of memory each).
SHAPE_CASES = {
    "shape_7b_f16": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, d=4096, n_ff=11008, n_head=32, n_head_kv=32,
                                    rank=1024, n_vocab=1024, firing=0.10, seed=21),
    "shape_falcon40b_f16": synth.ModelSpec(arch=synth.ARCH_FALCON, wtype=synth.F16, d=8192, n_ff=32768, n_head=128, n_head_kv=8,
                                           rank=1024, n_vocab=1024, firing=0.10, seed=22),
    "shape_70b_q4_0": synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.Q4_0, d=8192, n_ff=28672, n_head=64, n_head_kv=8,
                                      rank=1024, n_vocab=1024, firing=0.12, seed=23),
    "shape_opt175b_f16": synth.ModelSpec(arch=synth.ARCH_OPT, wtype=synth.F16, d=12288, n_ff=49152, n_head=96, n_head_kv=96,
                                         rank=1536, n_vocab=1024, firing=0.08, norm_eps=0.0, seed=24),
}
ALL_CASES = {**MODEL_CASES, **SHAPE_CASES}


def prompt_for(spec):
    return np.random.default_rng(spec.seed + 1000).integers(3, spec.n_vocab, N_PROMPT).astype(np.int32)


def op_cases():
    """name -> dict(wtype, d, F, T, firing, seed, kind).  Tests regenerate inputs with `op_inputs`."""
    cases = {}
    for wt, wn in ((synth.F16, "f16"), (synth.Q4_0, "q4_0")):
        for T in (1, 4):
            for kind in ("zipf", "empty", "full", "single", "tail"):
                if T == 4 and kind not in ("zipf", "single"):
                    continue
                cases[f"{wn}_T{T}_{kind}"] = dict(wtype=wt, d=256, F=1280, T=T, kind=kind, seed=len(cases) + 1)
        cases[f"{wn}_T1_wide"] = dict(wtype=wt, d=1024, F=2048, T=1, kind="zipf", seed=100 + wt)
    return cases


def op_inputs(c):
    rng = np.random.default_rng(c["seed"])
    d, F, T = c["d"], c["F"], c["T"]
    x = rng.standard_normal((T, d), dtype=np.float32)
    Wf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    Wtf = rng.standard_normal((F, d), dtype=np.float32) * np.float32(0.02)
    if c["wtype"] == synth.Q4_0:
        W, Wt = synth.quantize_q4_0(Wf), synth.quantize_q4_0(Wtf)
    else:
        W, Wt = Wf.astype(np.float16), Wtf.astype(np.float16)
    kind = c["kind"]
    if kind == "zipf":
        p = synth.zipf_profile(F, 0.15)[rng.permutation(F)]
        idx = np.where(rng.random((T, F)) < p, 1.0, -1.0)
        idx = idx * rng.random((T, F))          # logits of varying magnitude, some exactly +-0
    elif kind == "empty":
        idx = -np.ones((T, F))
    elif kind == "full":
        idx = np.ones((T, F))
    elif kind == "single":
        idx = -np.ones((T, F))
        idx[np.arange(T), rng.integers(0, F, T)] = 0.0   # logit == threshold counts as active
    else:  # tail: only the last rows
        idx = -np.ones((T, F))
        idx[:, -5:] = 2.0
    return x, W, Wt, idx.astype(np.float32)


def write_gguf(spec, tensors, path):
    """Write a PowerInfer GGUF the reference loader accepts (magic PWRI, ggml.c:19481-19495)."""
    from powerinfer_b200 import gguf_loader
    gguf_loader.write_model_file(spec, tensors, path)


def run_ref_decode(gguf_path, tokens, n_prompt, n_steps, n_vocab, mode="batch", forced=False, threads=1):
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_decode")
    with tempfile.TemporaryDirectory() as td:
        tp, op = os.path.join(td, "tok.i32"), os.path.join(td, "out.f32")
        np.asarray(tokens, np.int32).tofile(tp)
        cmd = [exe, gguf_path, tp, str(n_prompt), str(n_steps), str(threads), op, mode] + (["forced"] if forced else [])
        r = subprocess.run(cmd, check=True, capture_output=True, text=True)
        greedy = np.array([int(t) for t in r.stdout.split()], np.int32)
        logits = np.fromfile(op, np.float32).reshape(n_steps, n_vocab)
    return logits, greedy


def write_op_fixtures(ref):
    out = {}
    for name, c in op_cases().items():
        x, W, Wt, idx = op_inputs(c)
        up = ref.mul_mat_idx(c["wtype"], W, c["F"], c["d"], x, idx)
        h = np.maximum(up, 0)
        out[name + ".up"] = up
        out[name + ".down"] = ref.axpy(c["wtype"], Wt, c["F"], c["d"], h, idx)
        out[name + ".dense"] = ref.mul_mat(c["wtype"], W, c["F"], c["d"], x)
    rng = np.random.default_rng(7)
    xs = rng.standard_normal((3, 512), dtype=np.float32)
    out["rms_norm"] = ref.rms_norm(xs, 1e-5)
    out["norm"] = ref.norm(xs, 1e-5)
    sm = xs.copy()
    sm[:, 400:] = -np.inf
    out["soft_max"] = ref.soft_max(sm)
    for pos in (0, 1, 37, 300):
        out[f"rope_{pos}"] = ref.rope(xs[0], 128, 4, pos, 10000.0, False)
        out[f"rope_neox_{pos}"] = ref.rope(xs[0], 64, 8, pos, 10000.0, True)
    out["q8_0"] = ref.quantize_q8_0(xs)
    out["q4_0"] = ref.quantize_q4_0(xs * 0.02)
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **out)
    print("ops.npz:", len(out), "arrays")


def main():
    from oracle import pio
    only = set(sys.argv[1:])          # cases to (re)generate; none named: the op fixtures and the small models;
    if "shapes" in only:              # `shapes`: the configuration-shaped models
        only = (only - {"shapes"}) | set(SHAPE_CASES)
    if not only:
        write_op_fixtures(pio.Ref())
    for name, spec in (ALL_CASES if only else MODEL_CASES).items():
        if only and name not in only:
            continue
        tensors = synth.build_model(spec)
        prompt = prompt_for(spec)
        with tempfile.TemporaryDirectory() as td:
            path = os.path.join(td, name + ".powerinfer.gguf")
            write_gguf(spec, tensors, path)
            logits, greedy = run_ref_decode(path, prompt, N_PROMPT, N_STEPS, spec.n_vocab, "batch")
            logits_s, greedy_s = run_ref_decode(path, prompt, N_PROMPT, N_STEPS, spec.n_vocab, "single")
        same = np.array_equal(logits, logits_s)
        print(f"{name}: greedy {greedy[:8]}..., batch-prompt == token-by-token prompt: {same}")
        np.savez_compressed(os.path.join(HERE, f"model_{name}.npz"), logits=logits, greedy=greedy, prompt=prompt,
                            digest=np.array(synth.digest(tensors)), single_equals_batch=np.array(same))


if __name__ == "__main__":
    main()
