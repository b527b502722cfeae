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


def _s(b: bytes) -> bytes:
    return len(b).to_bytes(8, "little") + b


def test_extents_whose_product_wraps_64_bits_are_refused(tmp_path):
    """Four extents of 2^16 x 2^16 x 2^16 x 2^16 (each far below the per-extent limit) make an element count of 2^64,
    which wraps to 0: such an entry must be refused, not read as an empty tensor that advertises huge extents."""
    import struct
    for ne in ([1 << 16] * 4, [1 << 40, 1 << 24, 1, 1], [1 << 31, 1 << 31, 2, 1]):
        head = b"GGUF" + struct.pack("<I", 3) + struct.pack("<Q", 1) + struct.pack("<Q", 0)
        info = _s(b"big") + struct.pack("<I", 4) + b"".join(struct.pack("<Q", e) for e in ne) + struct.pack("<I", 0) + struct.pack("<Q", 0)
        blob = head + info
        blob += b"\0" * ((-len(blob)) % 32) + b"\0" * 64
        p = tmp_path / "wrap.gguf"
        p.write_bytes(blob)
        with pytest.raises(_lib.PiError):
            model_file.ModelFile(str(p))


def _random_container(rng):
    """A random GGUF v3 container: every key type (arrays of scalars and of strings included), tensors of the four types
    the readers know with 1..4 dimensions, a random alignment.  -> (bytes, expected keys, expected tensors)."""
    import struct
    fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
    lim = {0: (0, 255), 1: (-128, 127), 2: (0, 65535), 3: (-32768, 32767), 4: (0, 2**32 - 1), 5: (-2**31, 2**31 - 1),
           10: (0, 2**63 - 1), 11: (-2**63, 2**63 - 1)}

    def scalar(t):
        if t in lim:
            v = int(rng.integers(lim[t][0], lim[t][1], endpoint=True))
        elif t == 7:
            v = bool(rng.integers(0, 2))
        else:
            v = float(np.float32(rng.standard_normal()))
        return v, struct.pack(fmt[t], v)

    align = int(rng.choice([16, 32, 64, 256]))
    kvs, want_kv = [("general.alignment", 4, struct.pack("<I", align))], {"general.alignment": align}
    for i in range(int(rng.integers(3, 12))):
        key, t = f"k{i}.{'x' * int(rng.integers(0, 9))}", int(rng.choice([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]))
        if t == 8:
            v = bytes(rng.integers(97, 123, int(rng.integers(0, 20))).astype(np.uint8))
            kvs.append((key, t, _s(v))); want_kv[key] = v.decode()
        elif t == 9:
            et, n = int(rng.choice([0, 4, 5, 6, 8, 10])), int(rng.integers(0, 6))
            if et == 8:
                items = [bytes(rng.integers(97, 123, int(rng.integers(0, 7))).astype(np.uint8)) for _ in range(n)]
                kvs.append((key, t, struct.pack("<IQ", et, n) + b"".join(_s(x) for x in items))); want_kv[key] = [x.decode() for x in items]
            else:
                vals = [scalar(et) for _ in range(n)]
                kvs.append((key, t, struct.pack("<IQ", et, n) + b"".join(b for _, b in vals))); want_kv[key] = [v for v, _ in vals]
        else:
            v, b = scalar(t)
            kvs.append((key, t, b)); want_kv[key] = v
    tensors, blobs, off = [], [], 0
    for i in range(int(rng.integers(1, 7))):
        ty = int(rng.choice([0, 1, 2, 18]))
        nd = int(rng.integers(1, 5))
        ne = [int(rng.integers(1, 5)) for _ in range(nd)]
        if ty == 2:
            ne[0] = 32 * int(rng.integers(1, 4))
        n = int(np.prod(ne))
        nbytes = {0: n * 4, 1: n * 2, 2: n // 32 * 18, 18: n * 4}[ty]
        data = bytes(rng.integers(0, 256, nbytes).astype(np.uint8))
        tensors.append((f"t{i}", ne, ty, off, data))
        pad = (-nbytes) % align
        blobs.append(data + b"\0" * pad)
        off += nbytes + pad
    head = b"PWRI" + struct.pack("<IQQ", 3, len(tensors), len(kvs))
    for key, t, payload in kvs:
        head += _s(key.encode()) + struct.pack("<I", t) + payload
    for name, ne, ty, o, _ in tensors:
        head += _s(name.encode()) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", e) for e in ne) + struct.pack("<IQ", ty, o)
    head += b"\0" * ((-len(head)) % align)
    return head + b"".join(blobs), want_kv, tensors


def test_random_containers_read_the_same_by_both_readers(tmp_path):
    rng = np.random.default_rng(11)
    path = tmp_path / "r.gguf"
    for _ in range(60):
        blob, want_kv, want_t = _random_container(rng)
        path.write_bytes(blob)
        _, kv, tens = gguf_loader.read_gguf(str(path))
        for k, v in want_kv.items():
            if isinstance(v, float) or (isinstance(v, list) and v and isinstance(v[0], float)):
                assert np.allclose(kv[k], v, rtol=1e-6), k
            else:
                assert kv[k] == v, (k, kv[k], v)
        with model_file.ModelFile(str(path)) as f:
            for k, v in want_kv.items():
                if isinstance(v, str):
                    assert f.string(k) == v
                elif isinstance(v, bool) or (isinstance(v, int) and v >= 0):
                    assert f.u64(k) == int(v)
                elif isinstance(v, float):
                    assert np.float32(f.f32(k)) == np.float32(v)
                elif isinstance(v, int):
                    with pytest.raises(_lib.PiError, match="negative"):
                        f.u64(k)
            got = f.tensors()
            assert list(got) == [t[0] for t in want_t]
            for name, ne, ty, _, data in want_t:
                gty, gne, raw = got[name]
                assert gty == ty and list(gne) == ne + [1] * (4 - len(ne))
                assert raw.tobytes() == data
                assert np.ascontiguousarray(tens[name]).tobytes() == data
                assert tens[name].shape == (tuple(reversed(ne)) if ty != 2 else tuple(reversed(ne[1:])) + (ne[0] // 32 * 18,))
