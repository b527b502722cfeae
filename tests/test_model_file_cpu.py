"""The native reader for model and placement files (pi_model_file_*, host only) against the numpy reader and the specs
the files were written from; malformed files must come back as errors."""
import numpy as np
import pytest

import make_golden as mg
from powerinfer_b200 import _lib, gguf_loader, model_file, placement, synth
from powerinfer_b200.engine import PI_ARCH_BAMBOO


@pytest.mark.parametrize("name", sorted(mg.MODEL_CASES))
def test_native_reader_agrees_with_the_numpy_reader(tmp_path, name):
    pytest.importorskip("gguf")
    spec = mg.MODEL_CASES[name]
    path = str(tmp_path / "m.powerinfer.gguf")
    mg.write_gguf(spec, synth.build_model(spec), path)
    _, kv, tensors = gguf_loader.read_gguf(path)
    with model_file.ModelFile(path) as f:
        assert f.is_powerinfer
        assert f.string("general.architecture") == spec.arch_name
        got = f.tensors()
        assert sorted(got) == sorted(tensors)
        for tname, a in tensors.items():
            ty, ne, raw = got[tname]
            want_type = {np.dtype(np.float32): 0, np.dtype(np.float16): 1, np.dtype(np.uint8): 2, np.dtype(np.int32): 18}[a.dtype]
            assert ty == want_type, tname
            assert raw.tobytes() == np.ascontiguousarray(a).tobytes(), tname
            assert f.tensor(tname)[1] == ne
            rows = a.shape[0] if a.ndim == 2 else 1
            cols = ne[0]
            assert (ne[1] if a.ndim == 2 else 1) == rows and (cols == a.shape[-1] or a.dtype == np.uint8 and cols // 32 * 18 == a.shape[-1])
        cfg = f.engine_config()
        assert cfg.arch == (PI_ARCH_BAMBOO if spec.gate_sym else spec.arch)
        assert cfg.wtype == (_lib.PI_TYPE_Q4_0 if spec.wtype == synth.Q4_0 else _lib.PI_TYPE_F16)
        for k, v in dict(n_layer=spec.n_layer, d=spec.d, n_ff=spec.n_ff, n_head=spec.n_head, n_head_kv=spec.n_head_kv,
                         rank=spec.rank, n_vocab=spec.n_vocab, max_batch=1, n_ranks=1, rank_id=0).items():
            assert getattr(cfg, k) == v, k
        assert np.float32(cfg.norm_eps) == np.float32(spec.norm_eps) and cfg.threshold == np.float32(spec.threshold)
        if spec.arch != synth.ARCH_OPT:
            assert cfg.rope_base == np.float32(spec.rope_base) and cfg.n_pos == 0
        else:
            assert cfg.n_pos == synth.OPT_N_POS
        # the engine accepts what the reader made (sizes only: no device needed)
        from powerinfer_b200.engine import lib as elib
        import ctypes as C
        assert elib.pi_engine_workspace_bytes(C.byref(cfg)) > 0
        with pytest.raises(_lib.PiError):
            f.u64("general.architecture")                          # a string is not an integer
        with pytest.raises(_lib.PiError):
            f.tensor("blk.99.nope")


def test_placement_file_through_the_native_reader(tmp_path):
    rng = np.random.default_rng(3)
    counts = [rng.integers(0, 1000, 256) for _ in range(3)]
    pairs = [placement.gpu_idx_and_bucket(c, k) for c, k in zip(counts, (64, 0, 128))]
    path = str(tmp_path / "m.generated.gpuidx")
    gguf_loader.write_gpu_split(path, [p[0] for p in pairs], [p[1] for p in pairs], 7 << 30)
    with model_file.ModelFile(path) as f:
        assert f.is_powerinfer and f.string("general.architecture") == "generic.gpu_index"
        assert f.u64("split.vram_capacity") == 7 << 30 and f.u64("generic.gpu_index.block_count") == 3
        for i, (gi, gb) in enumerate(pairs):
            ty, ne, raw = f.tensor(f"blk.{i}.gpu_idx")
            assert ty == 18 and ne[0] == 256 and np.array_equal(raw.view(np.int32), gi)
            ty, ne, raw = f.tensor(f"blk.{i}.gpu_bucket")
            assert ty == 18 and ne[0] == len(gb) and (raw is None or np.array_equal(raw.view(np.int32), gb))
        with pytest.raises(_lib.PiError, match="generic.gpu_index is not one of"):
            f.engine_config()                                      # a placement file is not a model


def test_malformed_files_are_errors_not_faults(tmp_path):
    pytest.importorskip("gguf")
    spec = mg.MODEL_CASES["llama_f16"]
    good = tmp_path / "good.gguf"
    mg.write_gguf(spec, synth.build_model(spec), str(good))
    blob = good.read_bytes()
    cases = {"empty": b"", "short": blob[:10], "magic": b"NOPE" + blob[4:], "version": blob[:4] + (9).to_bytes(4, "little") + blob[8:],
             "kv_cut": blob[:200], "dir_cut": blob[:40000], "data_cut": blob[: len(blob) - 4096],
             "huge_counts": blob[:8] + (1 << 60).to_bytes(8, "little") + blob[16:]}
    rng = np.random.default_rng(0)
    for i in range(20):                                            # random corruption of the metadata region
        b = bytearray(blob[:60000])
        for p in rng.integers(8, len(b), 6):
            b[p] = int(rng.integers(0, 256))
        cases[f"fuzz{i}"] = bytes(b) + blob[60000:]
    for tag, data in cases.items():
        p = tmp_path / f"{tag}.gguf"
        p.write_bytes(data)
        try:
            with model_file.ModelFile(str(p)) as f:                # a corruption that leaves the structure intact may still open
                f.tensors()
                try:
                    f.engine_config()
                except _lib.PiError:
                    pass
            assert tag.startswith("fuzz"), tag                     # the deliberate breaks must all be refused
        except _lib.PiError:
            pass
    with pytest.raises(_lib.PiError, match="cannot open"):
        model_file.ModelFile(str(tmp_path / "missing.gguf"))
