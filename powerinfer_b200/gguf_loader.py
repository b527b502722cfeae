"""Reader for PowerInfer GGUF model files and reader / writer for the neuron-placement ("GPU index") files.

A PowerInfer model file is GGUF v3 with the magic `PWRI` instead of `GGUF` (ggml.h:247, ggml.c:19481-19495) and three
extra tensors per layer next to the usual ones: `blk.i.ffn_down_t.weight` (down transposed: one row per neuron),
`blk.i.fc1.weight`, `blk.i.fc2.weight` (the activation predictor), plus the key `powerinfer.sparse_threshold`
(llama.cpp:3159-3390).  The placement file written by powerinfer-py/powerinfer/export_split.py:54-76 is again GGUF with
magic `PWRI`, architecture `generic.gpu_index`, `blk.i.gpu_idx` / `blk.i.gpu_bucket` int32 tensors and
`split.vram_capacity`; llama.cpp:2781-2871 reads it back.

Only what the decode path needs is parsed: the header, the key/value table, the tensor directory, and F32 / F16 / Q4_0 /
I32 tensor data (returned as numpy views on a memory map, numpy shape = ggml `ne` reversed; Q4_0 as the raw block bytes
`[rows, cols/32*18]`, which is what powerinfer_b200.ggml_ops.upload_weight and the engine take).
"""
from __future__ import annotations

import mmap
import struct

import numpy as np

from . import synth

GGML_F32, GGML_F16, GGML_Q4_0, GGML_I32 = 0, 1, 2, 18          # enum ggml_type (ggml.h:307-333)
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self):
        n = self.take("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype):
        if vtype in _SCALAR:
            return self.take(_SCALAR[vtype])
        if vtype == _STRING:
            return self.string()
        if vtype == _ARRAY:
            etype, n = self.take("<I"), self.take("<Q")
            if etype in _SCALAR:                                   # bulk read: token scores / types are long
                fmt = _SCALAR[etype][1]
                size = struct.calcsize("<" + fmt)
                out = np.frombuffer(self.buf, dtype=np.dtype("<" + fmt), count=n, offset=self.pos).tolist()
                self.pos += n * size
                return out
            return [self.value(etype) for _ in range(n)]
        raise ValueError(f"gguf: unknown value type {vtype}")


def read_gguf(path: str):
    """-> (magic, kv dict, tensors dict name -> numpy array).  The arrays are views on a read-only memory map.
    A truncated or corrupt file raises ValueError."""
    try:
        return _read_gguf(path)
    except (struct.error, IndexError, OverflowError, MemoryError, TypeError, UnicodeError) as e:
        raise ValueError(f"{path}: malformed GGUF file ({type(e).__name__}: {e})") from e


def _read_gguf(path: str):
    f = open(path, "rb")
    mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    c = _Cursor(mm)
    magic = bytes(mm[0:4])
    if magic not in (b"PWRI", b"GGUF"):
        raise ValueError(f"{path}: not a GGUF / PowerInfer file (magic {magic!r})")
    c.pos = 4
    version = c.take("<I")
    if version not in (2, 3):
        raise ValueError(f"{path}: GGUF version {version} is not supported")
    n_tensors, n_kv = c.take("<Q"), c.take("<Q")
    kv = {}
    for _ in range(n_kv):
        key = c.string()
        kv[key] = c.value(c.take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = c.string()
        nd = c.take("<I")
        ne = [c.take("<Q") for _ in range(nd)]
        ttype, off = c.take("<I"), c.take("<Q")
        infos.append((name, ne, ttype, off))
    align = int(kv.get("general.alignment", 32))
    base = (c.pos + align - 1) // align * align
    tensors = {}
    for name, ne, ttype, off in infos:
        shape = tuple(reversed(ne))                                # ne[0] is the fastest dimension
        n = int(np.prod(ne)) if ne else 1
        if ttype == GGML_F32:
            a = np.frombuffer(mm, np.float32, n, base + off).reshape(shape)
        elif ttype == GGML_F16:
            a = np.frombuffer(mm, np.float16, n, base + off).reshape(shape)
        elif ttype == GGML_I32:
            a = np.frombuffer(mm, np.int32, n, base + off).reshape(shape)
        elif ttype == GGML_Q4_0:
            if ne[0] % 32:
                raise ValueError(f"{name}: Q4_0 row of {ne[0]} values")
            a = np.frombuffer(mm, np.uint8, n // 32 * 18, base + off).reshape(shape[:-1] + (ne[0] // 32 * 18,))
        else:
            raise ValueError(f"{name}: ggml type {ttype} is not on the decode path (F32, F16, Q4_0, I32 are)")
        tensors[name] = a
    return magic, kv, tensors


# "bamboo" is the llama graph with the symmetric gate (llama.cpp:2354-2355, 5028)
_ARCH = {"llama": synth.ARCH_LLAMA, "bamboo": synth.ARCH_LLAMA, "falcon": synth.ARCH_FALCON, "opt": synth.ARCH_OPT}


def load_model(path: str):
    """A PowerInfer GGUF -> (ModelSpec, tensors) in the form powerinfer_b200.engine.DecodeEngine takes.

    Hyper-parameters follow llm_load_hparams (llama.cpp:2330-2400): `<arch>.embedding_length`, `.block_count`,
    `.feed_forward_length`, `.attention.head_count(_kv)`, the norm epsilon key of the architecture, `.rope.freq_base`,
    `powerinfer.sparse_threshold`; the vocabulary size is the row count of `token_embd.weight`, the predictor rank the row
    count of `blk.0.fc1.weight`.  The 2-D weights must all be F16 or all Q4_0 (predictors may stay F16)."""
    magic, kv, t = read_gguf(path)
    arch_name = kv.get("general.architecture")
    if arch_name not in _ARCH:
        raise ValueError(f"{path}: architecture {arch_name!r} is not one of llama / bamboo / falcon / opt")
    for need in ("blk.0.ffn_down_t.weight", "blk.0.fc1.weight", "blk.0.fc2.weight"):
        if need not in t:
            raise ValueError(f"{path}: {need} is missing: not a PowerInfer (sparse) model file")
    arch = _ARCH[arch_name]
    k = lambda s, default=None: kv.get(f"{arch_name}.{s}", default)
    n_head = int(k("attention.head_count"))
    up = t["blk.0.ffn_up.weight"]
    wtype = synth.Q4_0 if up.dtype == np.uint8 else synth.F16
    d = int(k("embedding_length"))
    eps_key = "attention.layer_norm_rms_epsilon" if arch == synth.ARCH_LLAMA else "attention.layer_norm_epsilon"
    eps = float(k(eps_key, 1e-5 if arch != synth.ARCH_OPT else 0.0))
    spec = synth.ModelSpec(arch=arch, wtype=wtype, n_layer=int(k("block_count")), d=d, n_ff=int(k("feed_forward_length")),
                           n_head=n_head, n_head_kv=int(k("attention.head_count_kv", n_head)),
                           rank=int(t["blk.0.fc1.weight"].shape[0]), n_vocab=int(t["token_embd.weight"].shape[0]),
                           n_ctx=int(k("context_length", 512)), norm_eps=eps, rope_base=float(k("rope.freq_base", 10000.0)),
                           threshold=float(kv.get("powerinfer.sparse_threshold", 0.0)),
                           falcon_two_norms="blk.0.attn_norm_2.weight" in t, gate_sym=arch_name == "bamboo")
    return spec, t


def load_gpu_split(path: str):
    """A `.generated.gpuidx` placement file -> (list of gpu_idx int32 [F], list of gpu_bucket int32 [k], vram_capacity)."""
    magic, kv, t = read_gguf(path)
    n = int(kv.get("generic.gpu_index.block_count", 0)) or len([k for k in t if k.endswith(".gpu_idx")])
    idx = [np.asarray(t[f"blk.{i}.gpu_idx"]) for i in range(n)]
    bucket = [np.asarray(t[f"blk.{i}.gpu_bucket"]) for i in range(n)]
    return idx, bucket, int(kv.get("split.vram_capacity", 0))


def _wstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gpu_split(path: str, gpu_idx: list, gpu_bucket: list, vram_capacity: int) -> None:
    """The file export_split.py:54-76 writes: architecture `generic.gpu_index`, its block count, `split.vram_capacity`
    (u64), and per layer the int32 tensors `blk.i.gpu_idx` [F] and `blk.i.gpu_bucket` [k]; magic PWRI, version 3."""
    arch = "generic.gpu_index"
    kvs = [("general.architecture", 8, _wstr(arch)), (f"{arch}.block_count", 4, struct.pack("<I", len(gpu_idx))),
           ("split.vram_capacity", 10, struct.pack("<Q", int(vram_capacity)))]
    blobs, infos, off = [], [], 0
    for i, (gi, gb) in enumerate(zip(gpu_idx, gpu_bucket)):
        for name, a in ((f"blk.{i}.gpu_idx", gi), (f"blk.{i}.gpu_bucket", gb)):
            a = np.ascontiguousarray(a, dtype=np.int32)
            infos.append(_wstr(name) + struct.pack("<I", 1) + struct.pack("<Q", a.size) + struct.pack("<I", GGML_I32) + struct.pack("<Q", off))
            pad = (-a.nbytes) % 32
            blobs.append(a.tobytes() + b"\0" * pad)
            off += a.nbytes + pad
    head = b"PWRI" + struct.pack("<I", 3) + struct.pack("<Q", len(infos)) + struct.pack("<Q", len(kvs))
    for key, vt, payload in kvs:
        head += _wstr(key) + struct.pack("<I", vt) + payload
    head += b"".join(infos)
    head += b"\0" * ((-len(head)) % 32)
    with open(path, "wb") as f:
        f.write(head)
        for b in blobs:
            f.write(b)


def write_model_file(spec, tensors, path):
    """Write a synthetic model as a PowerInfer GGUF file the reference's loader accepts (magic PWRI, ggml.c:19481-19495; keys and
    tensor names as llm_load_hparams / llm_load_sparse_model_tensors read them, llama.cpp:2330-2400, 3159-3390).  Needs the
    `gguf` package."""
    from . import synth
    import gguf
    V = spec.n_vocab
    toks = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + [f"tok{i}" for i in range(V - 259)]
    types = [2, 3, 3] + [6] * 256 + [1] * (V - 259)
    arch = spec.arch_name
    w = gguf.GGUFWriter(path, arch)
    w.add_name("synthetic-" + arch)
    w.add_context_length(2050 if spec.arch == synth.ARCH_OPT else spec.n_ctx)
    w.add_embedding_length(spec.d)
    w.add_block_count(spec.n_layer)
    w.add_feed_forward_length(spec.n_ff)
    w.add_head_count(spec.n_head)
    w.add_head_count_kv(spec.n_head_kv)
    if spec.arch == synth.ARCH_LLAMA:
        w.add_rope_dimension_count(spec.head_dim)
        w.add_layer_norm_rms_eps(spec.norm_eps)
        w.add_rope_freq_base(spec.rope_base)
    elif spec.arch == synth.ARCH_FALCON:
        w.add_layer_norm_eps(spec.norm_eps)
        w.add_rope_freq_base(spec.rope_base)
    w.add_float32("powerinfer.sparse_threshold", spec.threshold)
    w.add_tokenizer_model("llama")
    w.add_token_list(toks)
    w.add_token_scores([0.0] * V)
    w.add_token_types(types)
    w.add_bos_token_id(1)
    w.add_eos_token_id(2)
    w.add_unk_token_id(0)
    for name, a in tensors.items():
        if name.startswith("_"):
            continue
        if a.dtype == np.uint8:     # Q4_0 block bytes [rows, cols/32*18]
            w.add_tensor(name, a, raw_dtype=gguf.GGMLQuantizationType.Q4_0)
        else:
            w.add_tensor(name, a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    with open(path, "r+b") as f:
        f.write(b"PWRI")
