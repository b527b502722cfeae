"""Neuron / head sharding of a PowerInfer model over the GPUs of one node (host-side logic, no CUDA needed).

The B200 analogue of the reference's gpu_idx / gpu_bucket placement (llama.cpp:2781-2997): each rank owns a contiguous
range of whole 32-neuron blocks of the FFN (rows of fc2, up, gate, down_t) and a contiguous range of attention heads (rows
of q / k / v, the matching columns of attn_output).  Whole 32-neuron blocks keep the Q4_0 axpy coefficients (quantised per
32 neurons) identical to the unsharded model; whole heads keep Q8_0 activation blocks (32 columns) intact.
"""
from __future__ import annotations

import numpy as np

from . import synth

try:                                    # torch tensors are accepted when torch is present
    import torch
except Exception:                       # pragma: no cover
    torch = None

PI_TYPE_Q4_0 = synth.Q4_0


def _is_torch(a):
    return torch is not None and isinstance(a, torch.Tensor)


def shard_rows(a, n_ranks: int, rank: int):
    n = a.shape[0] // n_ranks
    return a[rank * n:(rank + 1) * n]


def shard_cols(a, wtype: int, n_ranks: int, rank: int):
    """Column slice of a [rows, cols] weight: F16 elements, or Q4_0 block bytes (18 per 32 columns)."""
    unit = 18 if (wtype == PI_TYPE_Q4_0 and str(a.dtype).endswith('uint8')) else 1
    per = a.shape[1] // n_ranks
    assert per % unit == 0
    return a[:, rank * per:(rank + 1) * per]


def shard_layer(spec: synth.ModelSpec, t: dict, il: int, n_ranks: int, rank: int) -> dict:
    """The slice of layer `il` that rank `rank` holds: its FFN neurons (rows of fc2 / up / gate / down_t, a contiguous
    range of whole 32-neuron blocks) and its heads (rows of q/k/v, columns of attn_output).  Works on numpy arrays and
    torch tensors alike.  Returns the engine's tensor names (wqkv, bqkv, wo, ...)."""
    p = f"blk.{il}."
    cat = (lambda xs: torch.cat(xs, 0)) if _is_torch(t[p + "fc1.weight"]) else (lambda xs: np.concatenate(xs, 0))
    g = lambda k: t.get(p + k)
    d, dkv = spec.d, spec.d_kv
    out = {}
    for k in ("attn_norm.weight", "attn_norm.bias", "attn_norm_2.weight", "attn_norm_2.bias", "ffn_norm.weight", "ffn_norm.bias"):
        out[k] = g(k)
    if spec.arch == synth.ARCH_FALCON:
        w = g("attn_qkv.weight")
        q, k_, v = w[:d], w[d:d + dkv], w[d + dkv:]
        bq = bk = bv = None
    else:
        q, k_, v = g("attn_q.weight"), g("attn_k.weight"), g("attn_v.weight")
        bq, bk, bv = g("attn_q.bias"), g("attn_k.bias"), g("attn_v.bias")
    out["wqkv"] = cat([shard_rows(q, n_ranks, rank), shard_rows(k_, n_ranks, rank), shard_rows(v, n_ranks, rank)])
    out["bqkv"] = None if bq is None else cat([shard_rows(bq, n_ranks, rank), shard_rows(bk, n_ranks, rank), shard_rows(bv, n_ranks, rank)])
    out["wo"] = shard_cols(g("attn_output.weight"), spec.wtype, n_ranks, rank)
    out["bo"] = g("attn_output.bias")
    out["fc1"] = g("fc1.weight")
    out["fc2"] = shard_rows(g("fc2.weight"), n_ranks, rank)
    out["gate"] = None if g("ffn_gate.weight") is None else shard_rows(g("ffn_gate.weight"), n_ranks, rank)
    out["up"] = shard_rows(g("ffn_up.weight"), n_ranks, rank)
    out["down_t"] = shard_rows(g("ffn_down_t.weight"), n_ranks, rank)
    out["up_b"] = None if g("ffn_up.bias") is None else shard_rows(g("ffn_up.bias"), n_ranks, rank)
    out["down_b"] = g("ffn_down_t.bias")
    return out


