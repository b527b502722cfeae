"""Seeded synthetic models drawn directly on the GPU, one rank's slice at a time.

The full-size configurations (tens of GB of Q4_0) are never materialised on the host: each rank draws the
rows it owns with torch's CUDA generator, rounds them to FP16 as the configurations specify, quantises with the
library's Q4_0 kernel (the reference's model-file rule) and hands them to the engine already sharded.  The
firing profile of the bias-free predictor follows powerinfer_b200.synth (fc2 row i = w_i + c_i).
The draw depends on (seed, layer, tensor, rank), so an N-rank model is not the same draw as the 1-rank model;
for bit-identical sharding of one model use powerinfer_b200.synth + engine.shard_layer (small models, tests).
"""
from __future__ import annotations

import math

import torch

from . import synth
from ._lib import PI_TYPE_Q4_0, check, lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _randn16(gen, rows, cols, sigma):
    return (torch.randn(rows, cols, device="cuda", dtype=torch.float32, generator=gen) * sigma).to(torch.float16)


def _weight(gen, rows, cols, spec):
    """[rows, cols] weight in the spec's storage type: F16, or ggml Q4_0 block bytes [rows, cols/32*18]."""
    w = _randn16(gen, rows, cols, spec.sigma)
    if spec.wtype != PI_TYPE_Q4_0:
        return w
    out = torch.empty(rows, cols // 32 * 18, dtype=torch.uint8, device="cuda")
    wf = w.float()
    check(lib.pi_quantize_q4_0(wf.data_ptr(), out.data_ptr(), rows, cols, _stream()))
    torch.cuda.current_stream().synchronize()
    return out


def _vec(gen, n, kind):
    r = torch.randn(n, device="cuda", dtype=torch.float32, generator=gen)
    return 1.0 + 0.1 * r if kind == "w" else 0.02 * r


def build_globals(spec: synth.ModelSpec, seed: int) -> dict:
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed * 1000003 + 17)
    t = {"token_embd.weight": _randn16(gen, spec.n_vocab, spec.d, spec.sigma), "output_norm.weight": _vec(gen, spec.d, "w")}
    if spec.arch == synth.ARCH_OPT:
        t["position_embd.weight"] = _randn16(gen, synth.OPT_N_POS, spec.d, spec.sigma)
    if spec.arch != synth.ARCH_LLAMA:
        t["output_norm.bias"] = _vec(gen, spec.d, "b")
    if spec.arch != synth.ARCH_OPT:
        t["output.weight"] = _weight(gen, spec.n_vocab, spec.d, spec)
    return t


def build_local_layer(spec: synth.ModelSpec, il: int, n_ranks: int, rank: int, seed: int) -> dict:
    """Layer `il` as rank `rank` holds it, under the engine's tensor names (see engine.shard_layer)."""
    d, hd = spec.d, spec.head_dim
    dq, dkv, F = d // n_ranks, spec.d_kv // n_ranks, spec.n_ff // n_ranks
    gen = torch.Generator(device="cuda")
    gen.manual_seed((seed * 1000003 + il) * 64 + 1)          # replicated tensors: same on every rank
    out = {"attn_norm.weight": _vec(gen, d, "w")}
    if spec.arch != synth.ARCH_LLAMA:
        out["attn_norm.bias"] = _vec(gen, d, "b")
    if spec.arch == synth.ARCH_FALCON and spec.falcon_two_norms:
        out["attn_norm_2.weight"] = _vec(gen, d, "w")
        out["attn_norm_2.bias"] = _vec(gen, d, "b")
    if spec.arch != synth.ARCH_FALCON:
        out["ffn_norm.weight"] = _vec(gen, d, "w")
        if spec.arch == synth.ARCH_OPT:
            out["ffn_norm.bias"] = _vec(gen, d, "b")
    out["fc1"] = _randn16(gen, spec.rank, d, spec.sigma)
    if spec.arch == synth.ARCH_OPT:
        out["bo"] = _vec(gen, d, "b")
        out["down_b"] = _vec(gen, d, "b")
    # this rank's slice
    gen.manual_seed((seed * 1000003 + il) * 64 + 2 + rank)
    out["wqkv"] = _weight(gen, dq + 2 * dkv, d, spec)
    out["wo"] = _weight(gen, d, dq, spec)
    if spec.arch == synth.ARCH_OPT:
        out["bqkv"] = _vec(gen, dq + 2 * dkv, "b")
        out["up_b"] = _vec(gen, F, "b")
    if spec.arch == synth.ARCH_LLAMA:
        out["gate"] = _weight(gen, F, d, spec)
    out["up"] = _weight(gen, F, d, spec)
    out["down_t"] = _weight(gen, F, d, spec)
    # predictor output rows with the Zipf firing profile: ranks are a permutation of ALL neurons, this rank takes its range
    gperm = torch.Generator(device="cpu")
    gperm.manual_seed(seed * 7919 + il)
    ranks = torch.randperm(spec.n_ff, generator=gperm)[rank * F:(rank + 1) * F]
    profile = torch.from_numpy(synth.zipf_profile(spec.n_ff, spec.firing, spec.zipf_s))
    p = profile[ranks].clamp(1e-9, 1 - 1e-9)
    z = torch.special.ndtri(p)
    c = (spec.sigma * z / (0.564 * math.sqrt(spec.rank))).float().cuda()
    w = torch.randn(F, spec.rank, device="cuda", dtype=torch.float32, generator=gen) * spec.sigma
    out["fc2"] = (w + c[:, None]).to(torch.float16)
    return out


def build_local_model(spec: synth.ModelSpec, n_ranks: int = 1, rank: int = 0, seed: int = 0):
    layers = [build_local_layer(spec, il, n_ranks, rank, seed) for il in range(spec.n_layer)]
    return build_globals(spec, seed), layers
