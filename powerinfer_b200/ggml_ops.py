"""Host-side mirror of the reference's operator API for the hot path, on torch CUDA tensors.

Function names and argument meaning follow ggml.h (ggml_mul_mat_idx, ggml_axpy, ggml_mul_mat,
ggml_rms_norm, ggml_norm, ggml_rope_custom, ggml_soft_max + the KQV block) so that a test written
against the reference's graph builder reads the same here.  Every function calls the CUDA library
through its C ABI; torch only provides device memory and the current stream.

Shapes use the row-major view of ggml tensors: a ggml tensor with ne = {n, T} is a torch tensor
[T, n].  Weights are `Weight` objects made by `upload_weight` (the analogue of
ggml_cuda_transform_tensor): F16 rows, or Q4_0 blocks re-laid out for aligned 128-bit loads.
"""
from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import _lib
from ._lib import PI_TYPE_F16, PI_TYPE_Q4_0, check, lib

sparse_pred_threshold = 0.0        # ggml.h:2219 `extern float sparse_pred_threshold`


@dataclasses.dataclass
class Weight:
    wtype: int
    data: torch.Tensor             # uint8 device buffer: F16 rows or planar Q4_0 rows
    nrows: int
    ncols: int

    @property
    def ptr(self) -> int:
        return self.data.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


class Workspace:
    """Scratch for the operators below, grown on demand (the C ABI itself never allocates)."""

    def __init__(self):
        self.buf = None

    def get(self, ncols: int, nrows: int, T: int):
        need = lib.pi_workspace_bytes(ncols, nrows, T)
        if self.buf is None or self.buf.numel() < need:
            self.buf = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        off = (-self.buf.data_ptr()) % 256
        return self.buf.data_ptr() + off, self.buf.numel() - off


_ws = Workspace()


def last_op_status() -> int:
    """Status of the last sparse operator issued through this module (pi_op_status): 0, or 5 (a bounded device-side wait ran out)."""
    if _ws.buf is None:
        return 0
    off = (-_ws.buf.data_ptr()) % 256
    return int(lib.pi_op_status(_ws.buf.data_ptr() + off, _stream()))


def upload_weight(host: np.ndarray, wtype: int, nrows: int, ncols: int) -> Weight:
    """host: float16 [nrows, ncols], or uint8 ggml Q4_0 blocks [nrows, ncols/32*18]."""
    if wtype == PI_TYPE_F16:
        assert host.dtype == np.float16 and host.shape == (nrows, ncols)
        dev = torch.from_numpy(np.ascontiguousarray(host).view(np.uint8).reshape(-1)).cuda()
        return Weight(wtype, dev, nrows, ncols)
    raw = torch.from_numpy(np.ascontiguousarray(host, np.uint8).reshape(-1)).cuda()
    assert raw.numel() == nrows * (ncols // 32) * 18
    dev = torch.empty_like(raw)
    check(lib.pi_q4_0_repack(raw.data_ptr(), dev.data_ptr(), nrows, ncols, _stream()))
    return Weight(wtype, dev, nrows, ncols)


def quantize_q4_0(x: torch.Tensor) -> torch.Tensor:
    """F32 [rows, cols] on device -> ggml Q4_0 block bytes (uint8 [rows*cols/32*18])."""
    x = x.contiguous().float()
    out = torch.empty(x.numel() // 32 * 18, dtype=torch.uint8, device=x.device)
    check(lib.pi_quantize_q4_0(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _stream()))
    return out


def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous().float()
    out = torch.empty(x.numel() // 32 * 34, dtype=torch.uint8, device=x.device)
    check(lib.pi_quantize_q8_0(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _stream()))
    return out


def dequantize(w: Weight) -> torch.Tensor:
    if w.wtype == PI_TYPE_F16:
        return w.data.view(torch.float16).reshape(w.nrows, w.ncols).float()
    out = torch.empty(w.nrows, w.ncols, dtype=torch.float32, device="cuda")
    check(lib.pi_dequantize_q4_0(w.ptr, out.data_ptr(), w.nrows, w.ncols, _stream()))
    return out


def ggml_mul_mat(a: Weight, b: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """ggml_mul_mat(ctx, a, b): a [nrows, ncols] weights, b F32 [T, ncols] -> F32 [T, nrows]."""
    b = b.contiguous().float().reshape(-1, a.ncols)
    T = b.shape[0]
    dst = torch.empty(T, a.nrows, dtype=torch.float32, device="cuda")
    ws, wsn = _ws.get(a.ncols, a.nrows, T)
    check(lib.pi_mul_mat(a.wtype, a.ptr, a.nrows, a.ncols, b.data_ptr(), T, _p(bias), dst.data_ptr(), ws, wsn, _stream()))
    return dst


def ggml_mul_mat_idx(a: Weight, b: torch.Tensor, sparse_idx: torch.Tensor, gpu_bucket: torch.Tensor | None = None,
                     result_ne0: int | None = None) -> torch.Tensor:
    """ggml_mul_mat_idx / ggml_mul_mat_idx_upscale (ggml.h:1094-1106).

    a: rows of up / gate held on this device; b: F32 [T, ncols]; sparse_idx: F32 [T, F] predictor logits by
    global neuron id; gpu_bucket: int32 [a.nrows] global ids of a's rows (None: a holds all F rows);
    result_ne0: F when a bucket is given.  Returns F32 [T, F]."""
    b = b.contiguous().float().reshape(-1, a.ncols)
    T = b.shape[0]
    sparse_idx = sparse_idx.contiguous().float().reshape(T, -1)
    F = result_ne0 if gpu_bucket is not None else a.nrows
    assert F is not None and sparse_idx.shape[1] >= F
    dst = torch.empty(T, F, dtype=torch.float32, device="cuda")
    ws, wsn = _ws.get(a.ncols, max(a.nrows, F), T)
    check(lib.pi_mul_mat_idx(a.wtype, a.ptr, a.nrows, a.ncols, b.data_ptr(), T, sparse_idx.data_ptr(),
                             sparse_idx.shape[1], _p(gpu_bucket), sparse_pred_threshold, dst.data_ptr(), F,
                             ws, wsn, _stream()))
    return dst


def ggml_axpy(a: Weight, b: torch.Tensor, sparse_idx: torch.Tensor, hybrid_aux: torch.Tensor | None = None) -> torch.Tensor:
    """ggml_axpy (ggml.h:1107-1112): a = rows of ffn_down_t on this device, b = F32 [T, F] hidden activations,
    hybrid_aux = gpu_bucket (int32 [a.nrows]) or None.  Returns F32 [T, ncols]."""
    T = b.shape[0] if b.dim() == 2 else 1
    b = b.contiguous().float().reshape(T, -1)
    sparse_idx = sparse_idx.contiguous().float().reshape(T, -1)
    dst = torch.empty(T, a.ncols, dtype=torch.float32, device="cuda")
    ws, wsn = _ws.get(a.ncols, max(a.nrows, b.shape[1]), T)
    check(lib.pi_axpy(a.wtype, a.ptr, a.nrows, a.ncols, b.data_ptr(), T, b.shape[1], sparse_idx.data_ptr(),
                      sparse_idx.shape[1], _p(hybrid_aux), sparse_pred_threshold, dst.data_ptr(), ws, wsn, _stream()))
    return dst


def sparse_ffn(up: Weight, gate: Weight | None, down_t: Weight, x: torch.Tensor, sparse_idx: torch.Tensor,
               gpu_bucket: torch.Tensor | None = None, up_bias: torch.Tensor | None = None) -> torch.Tensor:
    """llm_build_ffn_sparse (llama.cpp:4652-4757) after the predictor, as one call: the two ggml_mul_mat_idx nodes, the
    relu / mul / bias nodes and ggml_axpy.  x F32 [T, d], sparse_idx F32 [T, F] -> F32 [T, d]."""
    x = x.contiguous().float().reshape(-1, up.ncols)
    T = x.shape[0]
    sparse_idx = sparse_idx.contiguous().float().reshape(T, -1)
    F = sparse_idx.shape[1]
    dst = torch.empty(T, up.ncols, dtype=torch.float32, device="cuda")
    ws, wsn = _ws.get(up.ncols, max(up.nrows, F), T)
    check(lib.pi_sparse_ffn(up.wtype, up.ptr, gate.ptr if gate is not None else None, down_t.ptr, up.nrows, up.ncols,
                            x.data_ptr(), T, sparse_idx.data_ptr(), F, _p(gpu_bucket), sparse_pred_threshold, _p(up_bias),
                            dst.data_ptr(), ws, wsn, _stream()))
    return dst


def predictor(fc1: Weight, fc2: Weight, p: torch.Tensor) -> torch.Tensor:
    """idx = mul_mat(fc2, relu(mul_mat(fc1, p))) (llama.cpp:4688-4695); p F32 [T, d] -> F32 [T, F]."""
    p = p.contiguous().float().reshape(-1, fc1.ncols)
    T = p.shape[0]
    idx = torch.empty(T, fc2.nrows, dtype=torch.float32, device="cuda")
    ws, wsn = _ws.get(max(fc1.ncols, fc2.ncols), max(fc1.nrows, fc2.nrows), T)
    check(lib.pi_predictor(fc1.ptr, fc2.ptr, fc1.ncols, fc1.nrows, fc2.nrows, p.data_ptr(), T, idx.data_ptr(), ws, wsn, _stream()))
    return idx


def active_list(sparse_idx: torch.Tensor):
    """Sorted ids of neurons whose logit >= threshold for at least one token, and their count (device tensors)."""
    sparse_idx = sparse_idx.contiguous().float()
    T, F = (sparse_idx.shape[0], sparse_idx.shape[1]) if sparse_idx.dim() == 2 else (1, sparse_idx.numel())
    lst = torch.empty(F, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws, wsn = _ws.get(F, F, T)
    check(lib.pi_active_list(sparse_idx.data_ptr(), F, T, F, sparse_pred_threshold, lst.data_ptr(), cnt.data_ptr(), ws, wsn, _stream()))
    return lst, cnt


def _norm(x, rms, eps, w, b):
    x = x.contiguous().float()
    x2 = x.reshape(-1, x.shape[-1])
    y = torch.empty_like(x2)
    check(lib.pi_norm(x2.data_ptr(), x2.shape[0], x2.shape[1], rms, eps, _p(w), _p(b), y.data_ptr(), _stream()))
    return y.reshape(x.shape)


def ggml_rms_norm(x, eps, w=None, b=None):
    """ggml_rms_norm followed by llm_build_norm's optional weight and bias."""
    return _norm(x, 1, eps, w, b)


def ggml_norm(x, eps, w=None, b=None):
    return _norm(x, 0, eps, w, b)


def rope_table(n_pos: int, head_dim: int, freq_base: float) -> torch.Tensor:
    host = np.empty((n_pos, head_dim // 2, 2), np.float32)
    lib.pi_rope_table_host(host.ctypes.data, n_pos, head_dim, freq_base)
    return torch.from_numpy(host).cuda()


def ggml_rope_custom(x: torch.Tensor, pos: torch.Tensor, n_dims: int, mode: int, table: torch.Tensor) -> torch.Tensor:
    """x F32 [T, n_heads, n_dims]; pos int32 [T]; mode 0 or 2 (neox)."""
    y = x.contiguous().float().clone()
    T, n_heads = y.shape[0], y.shape[1]
    check(lib.pi_rope(y.data_ptr(), T, n_heads, n_dims, pos.data_ptr(), table.data_ptr(), 1 if mode & 2 else 0, _stream()))
    return y


def attention_decode(q, k, v, k_cache, v_cache, pos, n_head, n_head_kv, seq=None):
    """KV store + KQV block for one new token per sequence.  q [T, n_head*hd], k/v [T, n_head_kv*hd] (RoPE'd),
    caches float16 [n_seq, n_ctx, n_head_kv*hd] updated in place.  Returns F32 [T, n_head*hd]."""
    T = q.shape[0]
    hd = q.shape[1] // n_head
    out = torch.empty(T, n_head * hd, dtype=torch.float32, device="cuda")
    check(lib.pi_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                  _p(seq), pos.data_ptr(), T, n_head, n_head_kv, hd, k_cache.shape[1], out.data_ptr(), _stream()))
    return out
