"""PowerInfer GGUF model files and placement files: what the loader reads is what the generator wrote (CPU only)."""
import dataclasses

import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import gguf_loader as gl
from powerinfer_b200 import placement, synth


@pytest.mark.parametrize("name", ["llama_q4_0", "llama_gqa_f16", "falcon_f16", "opt_f16", "bamboo_f16"])
def test_model_file_round_trip(tmp_path, name):
    pytest.importorskip("gguf")
    spec = mg.MODEL_CASES[name]
    t = synth.build_model(spec)
    path = str(tmp_path / "m.powerinfer.gguf")
    mg.write_gguf(spec, t, path)                          # the file the reference's llama.cpp loaded for the golden logits
    assert open(path, "rb").read(4) == b"PWRI"
    spec2, t2 = gl.load_model(path)
    a, b = dataclasses.asdict(spec), dataclasses.asdict(spec2)
    for k in ("arch", "gate_sym", "wtype", "n_layer", "d", "n_ff", "n_head", "n_head_kv", "rank", "n_vocab", "threshold", "rope_base"):
        assert a[k] == b[k], k
    assert np.float32(a["norm_eps"]) == np.float32(b["norm_eps"])
    assert synth.digest(t) == synth.digest({k: np.asarray(v) for k, v in t2.items()})
    q = t2["blk.0.ffn_up.weight"]
    assert q.shape == ((spec.n_ff, spec.d // 32 * 18) if spec.wtype == synth.Q4_0 else (spec.n_ff, spec.d))


def test_rejects_files_that_are_not_sparse_models(tmp_path):
    p = tmp_path / "x.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(ValueError, match="not a GGUF"):
        gl.read_gguf(str(p))
    pytest.importorskip("gguf")
    spec = mg.MODEL_CASES["llama_f16"]
    t = {k: v for k, v in synth.build_model(spec).items() if "fc1" not in k}
    path = str(tmp_path / "dense.gguf")
    mg.write_gguf(spec, t, path)
    with pytest.raises(ValueError, match="fc1"):
        gl.load_model(path)


def test_placement_file_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    L, F = 3, 1024
    counts = [np.floor(rng.pareto(1.2, F) * 10) for _ in range(L)]
    ks = placement.solve_gpu_split(counts, capacity=1024, batch=32, threshold=64)
    pairs = [placement.gpu_idx_and_bucket(c, k) for c, k in zip(counts, ks)]
    path = str(tmp_path / "m.gguf.generated.gpuidx")
    gl.write_gpu_split(path, [p[0] for p in pairs], [p[1] for p in pairs], vram_capacity=placement.vram_bytes(ks, 4608, 3))
    assert open(path, "rb").read(8) == b"PWRI" + (3).to_bytes(4, "little")
    idx, bucket, cap = gl.load_gpu_split(path)
    assert cap == sum(ks) * 4608 * 3 and len(idx) == L
    for (gi, gb), i2, b2, k in zip(pairs, idx, bucket, ks):
        assert np.array_equal(gi, i2) and np.array_equal(gb, b2) and b2.size == k and i2.sum() == k
    magic, kv, _ = gl.read_gguf(path)
    assert kv["general.architecture"] == "generic.gpu_index" and kv["generic.gpu_index.block_count"] == L


def test_corrupt_files_raise_value_error(tmp_path):
    pytest.importorskip("gguf")
    spec = mg.MODEL_CASES["llama_f16"]
    good = tmp_path / "good.gguf"
    mg.write_gguf(spec, synth.build_model(spec), str(good))
    blob = good.read_bytes()
    rng = np.random.default_rng(4)
    p = tmp_path / "bad.gguf"
    for i in range(150):
        if i % 2:
            data = blob[: int(rng.integers(1, len(blob)))]
        else:
            b = bytearray(blob[:60000])
            for q in rng.integers(4, len(b), 6):
                b[q] = int(rng.integers(0, 256))
            data = bytes(b) + blob[60000:]
        p.write_bytes(data)
        try:
            gl.read_gguf(str(p))
        except ValueError:
            pass
