"""ctypes bindings for the parity checker (TEST INFRASTRUCTURE ONLY).

`Oracle` wraps oracle/libpi_oracle.so, the plain-C restatement of the reference CPU
path; `Ref` wraps oracle/_ref/libpi_ref.so, the reference's own ggml CPU code compiled
unmodified.  Both take and return numpy arrays and expose the same method names so a
test can run either.  Nothing in the product package imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
F16, Q4_0 = 1, 2
ARCH_LLAMA, ARCH_FALCON, ARCH_OPT = 0, 1, 2

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_vp = C.c_void_p


def build(ref: bool = True) -> None:
    """Compile the checker (and, when the reference checkout is present, oracle/_ref)."""
    subprocess.run(["make", "-C", HERE, "-j8", "all" if ref else "libpi_oracle.so"], check=True,
                   stdout=subprocess.DEVNULL)


def _ptr(a):
    return a.ctypes.data_as(_vp) if a is not None else None


def row_bytes(wtype: int, n: int) -> int:
    return n // 32 * 18 if wtype == Q4_0 else n * 2


class _Base:
    """Shared numpy-level API; subclasses set self.lib and self.prefix."""

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def quantize_q4_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.size // 32 * 18, np.uint8)
        self._fn("quantize_q4_0" if self.prefix == "ref_" else "quantize_row_q4_0")(_ptr(x), _ptr(out), C.c_int64(x.size))
        return out

    def quantize_q8_0(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.size // 32 * 34, np.uint8)
        self._fn("quantize_q8_0" if self.prefix == "ref_" else "quantize_row_q8_0")(_ptr(x), _ptr(out), C.c_int64(x.size))
        return out

    def dequantize_q4_0(self, q, n):
        out = np.empty(n, np.float32)
        self._fn("dequantize_q4_0" if self.prefix == "ref_" else "dequantize_row_q4_0")(_ptr(q), _ptr(out), C.c_int64(n))
        return out

    def fp32_to_fp16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self._fn("fp32_to_fp16_row")(_ptr(x), _ptr(out), C.c_int64(x.size))
        return out


class Oracle(_Base):
    prefix = "pio_"

    def __init__(self):
        path = os.path.join(HERE, "libpi_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        self.lib = C.CDLL(path)
        self.lib.pio_vec_dot_f16.restype = C.c_float
        self.lib.pio_vec_dot_q4_0_q8_0.restype = C.c_float
        self.lib.pio_ctx_new.restype = _vp

    def mul_mat(self, wtype, W, nrows, ncols, x):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
        dst = np.empty((x.shape[0], nrows), np.float32)
        self.lib.pio_mul_mat(wtype, _ptr(W), C.c_int64(nrows), C.c_int64(ncols), _ptr(x), C.c_int64(x.shape[0]), _ptr(dst))
        return dst

    def mul_mat_idx(self, wtype, W, nrows, ncols, x, idx, gpu_idx=None, threshold=0.0):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
        idx = np.ascontiguousarray(idx, np.float32).reshape(x.shape[0], nrows)
        dst = np.empty((x.shape[0], nrows), np.float32)
        self.lib.pio_mul_mat_idx(wtype, _ptr(W), C.c_int64(nrows), C.c_int64(ncols), _ptr(x), C.c_int64(x.shape[0]),
                                 _ptr(idx), C.c_int64(nrows), _ptr(gpu_idx), C.c_float(threshold), _ptr(dst))
        return dst

    def axpy(self, wtype, Wt, nrows, ncols, h, idx, gpu_idx=None, threshold=0.0):
        h = np.ascontiguousarray(h, np.float32).reshape(-1, nrows)
        idx = np.ascontiguousarray(idx, np.float32).reshape(h.shape[0], nrows)
        dst = np.empty((h.shape[0], ncols), np.float32)
        self.lib.pio_axpy(wtype, _ptr(Wt), C.c_int64(nrows), C.c_int64(ncols), _ptr(h), C.c_int64(h.shape[0]),
                          _ptr(idx), C.c_int64(nrows), _ptr(gpu_idx), C.c_float(threshold), _ptr(dst))
        return dst

    def rms_norm(self, x, eps):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        for r in range(x.reshape(-1, x.shape[-1]).shape[0]):
            self.lib.pio_rms_norm(_ptr(x.reshape(-1, x.shape[-1])[r]), C.c_int64(x.shape[-1]), C.c_float(eps),
                                  _ptr(y.reshape(-1, x.shape[-1])[r]))
        return y

    def norm(self, x, eps):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        for r in range(x.reshape(-1, x.shape[-1]).shape[0]):
            self.lib.pio_norm(_ptr(x.reshape(-1, x.shape[-1])[r]), C.c_int64(x.shape[-1]), C.c_float(eps),
                              _ptr(y.reshape(-1, x.shape[-1])[r]))
        return y

    def soft_max(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        x2, y2 = x.reshape(-1, x.shape[-1]), y.reshape(-1, x.shape[-1])
        for r in range(x2.shape[0]):
            self.lib.pio_soft_max(_ptr(x2[r]), C.c_int64(x.shape[-1]), _ptr(y2[r]))
        return y

    def rope(self, x, head_dim, n_heads, pos, freq_base, neox):
        y = np.array(x, np.float32, copy=True).reshape(n_heads, head_dim)
        self.lib.pio_rope(_ptr(y), C.c_int64(head_dim), C.c_int64(n_heads), C.c_int32(pos), C.c_float(freq_base), int(neox))
        return y


class Ref(_Base):
    prefix = "ref_"

    def __init__(self):
        path = os.path.join(HERE, "_ref", "libpi_ref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path + " (run `make -C oracle` where the reference checkout is present)")
        self.lib = C.CDLL(path)
        for n in ("ref_mul_mat", "ref_mul_mat_idx", "ref_axpy"):
            getattr(self.lib, n).restype = C.c_double
        self.last_time = 0.0

    def mul_mat(self, wtype, W, nrows, ncols, x, n_threads=1, reps=1):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
        dst = np.empty((x.shape[0], nrows), np.float32)
        self.last_time = self.lib.ref_mul_mat(wtype, _ptr(W), C.c_int64(nrows), C.c_int64(ncols), _ptr(x),
                                              C.c_int64(x.shape[0]), _ptr(dst), n_threads, reps)
        return dst

    def mul_mat_idx(self, wtype, W, nrows, ncols, x, idx, gpu_idx=None, threshold=0.0, n_threads=1, reps=1):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, ncols)
        idx = np.ascontiguousarray(idx, np.float32).reshape(x.shape[0], nrows)
        if gpu_idx is None:   # the CPU op dereferences src[3] unconditionally (ggml.c:14211)
            gpu_idx = np.zeros(nrows, np.int32)
        dst = np.empty((x.shape[0], nrows), np.float32)
        self.last_time = self.lib.ref_mul_mat_idx(wtype, _ptr(W), C.c_int64(nrows), C.c_int64(ncols), _ptr(x),
                                                  C.c_int64(x.shape[0]), _ptr(idx), _ptr(gpu_idx), C.c_float(threshold),
                                                  _ptr(dst), n_threads, reps)
        return dst

    def axpy(self, wtype, Wt, nrows, ncols, h, idx, gpu_idx=None, threshold=0.0, n_threads=1, reps=1):
        h = np.ascontiguousarray(h, np.float32).reshape(-1, nrows)
        idx = np.ascontiguousarray(idx, np.float32).reshape(h.shape[0], nrows)
        if gpu_idx is None:   # NULL would skip every row in the F16 op (ggml.c:14424)
            gpu_idx = np.zeros(nrows, np.int32)
        dst = np.empty((h.shape[0], ncols), np.float32)
        self.last_time = self.lib.ref_axpy(wtype, _ptr(Wt), C.c_int64(nrows), C.c_int64(ncols), _ptr(h),
                                           C.c_int64(h.shape[0]), _ptr(idx), _ptr(gpu_idx), C.c_float(threshold),
                                           _ptr(dst), n_threads, reps)
        return dst

    def rms_norm(self, x, eps):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.ref_rms_norm(_ptr(x), C.c_int64(x.shape[-1]), C.c_int64(x.size // x.shape[-1]), C.c_float(eps), _ptr(y))
        return y

    def norm(self, x, eps):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.ref_norm(_ptr(x), C.c_int64(x.shape[-1]), C.c_int64(x.size // x.shape[-1]), C.c_float(eps), _ptr(y))
        return y

    def soft_max(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.lib.ref_soft_max(_ptr(x), C.c_int64(x.shape[-1]), C.c_int64(x.size // x.shape[-1]), _ptr(y))
        return y

    def rope(self, x, head_dim, n_heads, pos, freq_base, neox):
        x = np.ascontiguousarray(x, np.float32).reshape(n_heads, head_dim)
        y = np.empty_like(x)
        self.lib.ref_rope(_ptr(x), C.c_int64(head_dim), C.c_int64(n_heads), C.c_int32(pos), C.c_float(freq_base),
                          2 if neox else 0, _ptr(y))
        return y


class _Layer(C.Structure):
    _fields_ = [(n, _vp) for n in (
        "attn_norm_w", "attn_norm_b", "attn_norm2_w", "attn_norm2_b", "wq", "wk", "wv", "wo",
        "bq", "bk", "bv", "bo", "ffn_norm_w", "ffn_norm_b", "fc1", "fc2", "gate", "up", "down_t", "up_b", "down_b")]


class _Model(C.Structure):
    _fields_ = [("arch", C.c_int), ("wtype", C.c_int), ("n_layer", C.c_int), ("d", C.c_int), ("n_ff", C.c_int),
                ("n_head", C.c_int), ("n_head_kv", C.c_int), ("rank", C.c_int), ("n_vocab", C.c_int), ("n_ctx", C.c_int),
                ("norm_eps", C.c_float), ("rope_base", C.c_float), ("threshold", C.c_float),
                ("tok_embd", _vp), ("pos_embd", _vp), ("out_norm_w", _vp), ("out_norm_b", _vp), ("output", _vp),
                ("layers", C.POINTER(_Layer)), ("gate_sym", C.c_int)]


class OracleModel:
    """Whole-model decode through the C restatement, from a tensor dict of powerinfer_b200.synth.build_model."""

    def __init__(self, spec, tensors, oracle: "Oracle | None" = None):
        self.o = oracle or Oracle()
        self.spec, self.t = spec, tensors          # keep the arrays alive
        g = lambda k: _ptr(tensors[k]) if k in tensors else None
        self.layers = (_Layer * spec.n_layer)()
        for il in range(spec.n_layer):
            p, L = f"blk.{il}.", self.layers[il]
            L.attn_norm_w, L.attn_norm_b = g(p + "attn_norm.weight"), g(p + "attn_norm.bias")
            L.attn_norm2_w, L.attn_norm2_b = g(p + "attn_norm_2.weight"), g(p + "attn_norm_2.bias")
            if spec.arch == ARCH_FALCON:
                L.wq = g(p + "attn_qkv.weight")
            else:
                L.wq, L.wk, L.wv = g(p + "attn_q.weight"), g(p + "attn_k.weight"), g(p + "attn_v.weight")
                L.bq, L.bk, L.bv = g(p + "attn_q.bias"), g(p + "attn_k.bias"), g(p + "attn_v.bias")
            L.wo, L.bo = g(p + "attn_output.weight"), g(p + "attn_output.bias")
            L.ffn_norm_w, L.ffn_norm_b = g(p + "ffn_norm.weight"), g(p + "ffn_norm.bias")
            L.fc1, L.fc2 = g(p + "fc1.weight"), g(p + "fc2.weight")
            L.gate, L.up, L.down_t = g(p + "ffn_gate.weight"), g(p + "ffn_up.weight"), g(p + "ffn_down_t.weight")
            L.up_b, L.down_b = g(p + "ffn_up.bias"), g(p + "ffn_down_t.bias")
        self.m = _Model(spec.arch, spec.wtype, spec.n_layer, spec.d, spec.n_ff, spec.n_head, spec.n_head_kv,
                        spec.rank, spec.n_vocab, spec.n_ctx, spec.norm_eps, spec.rope_base, spec.threshold,
                        g("token_embd.weight"), g("position_embd.weight"), g("output_norm.weight"),
                        g("output_norm.bias"), g("output.weight"), self.layers, int(getattr(spec, "gate_sym", False)))
        self.ctx = _vp(self.o.lib.pio_ctx_new(C.byref(self.m)))

    def decode(self, token: int, pos: int, want_pred: bool = False):
        logits = np.empty(self.spec.n_vocab, np.float32)
        pred = np.empty((self.spec.n_layer, self.spec.n_ff), np.float32) if want_pred else None
        self.o.lib.pio_decode(self.ctx, C.c_int32(int(token)), C.c_int32(int(pos)), _ptr(logits), _ptr(pred))
        return (logits, pred) if want_pred else logits

    def decode_imposed(self, token: int, pos: int, idx_imposed):
        """decode() with every layer's sparse operators driven by the GIVEN predictor logits [n_layer, n_ff] (another
        implementation's); returns (logits, the predictor logits computed here)."""
        logits = np.empty(self.spec.n_vocab, np.float32)
        pred = np.empty((self.spec.n_layer, self.spec.n_ff), np.float32)
        imp = np.ascontiguousarray(idx_imposed, np.float32).reshape(self.spec.n_layer, self.spec.n_ff)
        self.o.lib.pio_decode_imposed(self.ctx, C.c_int32(int(token)), C.c_int32(int(pos)), _ptr(logits), _ptr(pred), _ptr(imp))
        return logits, pred

    def close(self):
        if self.ctx:
            self.o.lib.pio_ctx_free(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
