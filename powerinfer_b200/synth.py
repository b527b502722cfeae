"""Seeded synthetic PowerInfer models (host side, numpy).

The reference ships no checkpoints; every configuration it is measured on here is a
random-initialised model of a published shape.  This module draws such a model from a
seed so that the CUDA path, the CPU checker and a GGUF file written for the reference's
own loader all see identical bytes.

Tensor names and shapes follow what the reference's sparse loader requires
(llama.cpp:3238-3344: `blk.N.ffn_down_t`, `blk.N.fc1`, `blk.N.fc2`, ...): 2-D weights are
[rows, cols] with rows the output dimension; `ffn_down_t` is the down projection
transposed so that each neuron's output column is one contiguous row
(convert.py:1038-1048).

The reference's predictor has no bias (llama.cpp:4688-4692), so per-neuron firing rates
are obtained inside the same graph: fc2[i, :] = w_i + c_i, a constant added to the whole
row.  Because the predictor's hidden vector h = relu(fc1 p) is non-negative and sum(h)
/ |h| concentrates around 0.564 sqrt(R), c_i = sigma * Phi^-1(p_i) / (0.564 sqrt(R))
makes neuron i fire with probability close to p_i.  p_i follows a Zipf(s) rank profile
with the requested mean; ranks are a seeded permutation of the neurons.
"""
from __future__ import annotations

import dataclasses
import hashlib
import math
from statistics import NormalDist

import numpy as np

F16, Q4_0 = 1, 2
ARCH_LLAMA, ARCH_FALCON, ARCH_OPT = 0, 1, 2
OPT_N_POS = 2050
ARCH_NAMES = {ARCH_LLAMA: "llama", ARCH_FALCON: "falcon", ARCH_OPT: "opt"}


@dataclasses.dataclass
class ModelSpec:
    arch: int = ARCH_LLAMA
    wtype: int = F16
    n_layer: int = 2
    d: int = 256
    n_ff: int = 1280
    n_head: int = 4
    n_head_kv: int = 4
    rank: int = 64
    n_vocab: int = 512
    n_ctx: int = 128
    norm_eps: float = 1e-5
    rope_base: float = 10000.0
    threshold: float = 0.0
    firing: float = 0.10          # mean firing probability of the Zipf profile
    zipf_s: float = 1.1
    sigma: float = 0.02
    seed: int = 0
    falcon_two_norms: bool = True
    gate_sym: bool = False        # llama graph with the symmetric gate relu(gate) * relu(up): the reference's "bamboo"
                                  # architecture (llama.cpp:4732-4738, 5028); everything else is the llama graph

    @property
    def arch_name(self) -> str:
        """general.architecture of the model file the reference loads for this spec"""
        return "bamboo" if self.gate_sym else ARCH_NAMES[self.arch]

    @property
    def head_dim(self) -> int:
        return self.d // self.n_head

    @property
    def d_kv(self) -> int:
        return self.head_dim * self.n_head_kv


def zipf_profile(n: int, mean: float, s: float = 1.1, cap: float = 0.98) -> np.ndarray:
    """Per-rank firing probabilities p_r ~ r^-s rescaled to the given mean, clipped at `cap`."""
    w = np.arange(1, n + 1, dtype=np.float64) ** (-s)
    p = w * (mean * n / w.sum())
    for _ in range(64):                      # clip and give the excess back to the unclipped tail
        over = p > cap
        if not over.any():
            break
        excess = (p[over] - cap).sum()
        p[over] = cap
        free = ~over & (p < cap)
        p[free] += excess * p[free] / p[free].sum()
    return np.minimum(p, cap)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """Q4_0 blocks by the reference's model-file rule (ggml-quants.c:428-463), vectorised.

    Returns uint8 [rows, cols/32*18] in the ggml block layout {fp16 d; uint8 qs[16]}.
    """
    x = np.ascontiguousarray(x, np.float32)
    rows, cols = x.shape
    b = x.reshape(rows, cols // 32, 32)
    amax_i = np.abs(b).argmax(axis=2)                       # first index of the largest magnitude
    mx = np.take_along_axis(b, amax_i[..., None], axis=2)[..., 0]
    d = (mx / np.float32(-8)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1) / d, np.float32(0)).astype(np.float32)
    q = (b * inv[..., None]).astype(np.float32) + np.float32(8.5)
    q = np.minimum(q.astype(np.int8), 15).astype(np.uint8)  # C cast truncates toward zero, as astype does
    packed = (q[..., :16] | (q[..., 16:] << 4)).astype(np.uint8)
    out = np.empty((rows, cols // 32, 18), np.uint8)
    out[..., 0:2] = d.astype(np.float16).view(np.uint8).reshape(rows, cols // 32, 2)
    out[..., 2:] = packed
    return out.reshape(rows, cols // 32 * 18)


def build_model(spec: ModelSpec, fast_q4: bool = False) -> dict:
    """Draw every tensor of the model.  2-D weights are float16 arrays, or uint8 Q4_0 block
    arrays when spec.wtype == Q4_0 (predictor, embeddings and 1-D tensors stay F16 / F32).
    fast_q4 (timing runs on large shapes only, never parity): Q4_0 blocks are drawn directly (uniform nibbles under one
    scale chosen so that the weights' standard deviation is sigma) instead of quantising normal draws."""
    rng = np.random.default_rng(spec.seed)
    d, F, R, dkv = spec.d, spec.n_ff, spec.rank, spec.d_kv

    def f16(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(spec.sigma)).astype(np.float16)

    def w2(*shape):
        if spec.wtype == Q4_0 and fast_q4:
            rows, cols = shape
            out = rng.integers(0, 256, (rows, cols // 32, 18), dtype=np.uint8)
            out[..., 0:2] = np.array([spec.sigma / 4.61], np.float16).view(np.uint8)      # std of a uniform nibble - 8 is 4.61
            return out.reshape(rows, cols // 32 * 18)
        w = f16(*shape)
        return quantize_q4_0(w.astype(np.float32)) if spec.wtype == Q4_0 else w

    def vec(n, kind):
        if kind == "w":
            return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        return (0.02 * rng.standard_normal(n)).astype(np.float32)

    t: dict = {"token_embd.weight": f16(spec.n_vocab, d)}
    if spec.arch == ARCH_OPT:
        t["position_embd.weight"] = f16(OPT_N_POS, d)   # the loader fixes n_ctx_train = 2050 (llama.cpp:2369-2379)
    t["output_norm.weight"] = vec(d, "w")
    if spec.arch != ARCH_LLAMA:
        t["output_norm.bias"] = vec(d, "b")
    if spec.arch != ARCH_OPT:
        t["output.weight"] = w2(spec.n_vocab, d)

    kappa = 0.564 * math.sqrt(R)
    nd = NormalDist()
    profile = zipf_profile(F, spec.firing, spec.zipf_s)
    z_of_rank = np.array([nd.inv_cdf(float(p)) for p in profile], np.float64)
    firing = np.empty((spec.n_layer, F), np.float32)
    for il in range(spec.n_layer):
        p = f"blk.{il}."
        t[p + "attn_norm.weight"] = vec(d, "w")
        if spec.arch != ARCH_LLAMA:
            t[p + "attn_norm.bias"] = vec(d, "b")
        if spec.arch == ARCH_FALCON:
            if spec.falcon_two_norms:
                t[p + "attn_norm_2.weight"] = vec(d, "w")
                t[p + "attn_norm_2.bias"] = vec(d, "b")
            t[p + "attn_qkv.weight"] = w2(d + 2 * dkv, d)
        else:
            t[p + "attn_q.weight"] = w2(d, d)
            t[p + "attn_k.weight"] = w2(dkv, d)
            t[p + "attn_v.weight"] = w2(dkv, d)
            if spec.arch == ARCH_OPT:
                t[p + "attn_q.bias"] = vec(d, "b")
                t[p + "attn_k.bias"] = vec(dkv, "b")
                t[p + "attn_v.bias"] = vec(dkv, "b")
        t[p + "attn_output.weight"] = w2(d, d)
        if spec.arch == ARCH_OPT:
            t[p + "attn_output.bias"] = vec(d, "b")
        if spec.arch != ARCH_FALCON:
            t[p + "ffn_norm.weight"] = vec(d, "w")
            if spec.arch == ARCH_OPT:
                t[p + "ffn_norm.bias"] = vec(d, "b")
        if spec.arch == ARCH_LLAMA:
            t[p + "ffn_gate.weight"] = w2(F, d)
        t[p + "ffn_up.weight"] = w2(F, d)
        t[p + "ffn_down_t.weight"] = w2(F, d)
        if spec.arch == ARCH_OPT:
            t[p + "ffn_up.bias"] = vec(F, "b")
            t[p + "ffn_down_t.bias"] = vec(d, "b")
        t[p + "fc1.weight"] = f16(R, d)
        ranks = rng.permutation(F)                         # neuron i has Zipf rank ranks[i]
        c = (spec.sigma * z_of_rank[ranks] / kappa).astype(np.float32)
        w = rng.standard_normal((F, R), dtype=np.float32) * np.float32(spec.sigma)
        t[p + "fc2.weight"] = (w + c[:, None]).astype(np.float16)
        firing[il] = profile[ranks]
    t["_firing_profile"] = firing
    return t


def digest(tensors: dict) -> str:
    """SHA-256 over all tensor bytes in name order: pins a fixture to the exact weights it was made from."""
    h = hashlib.sha256()
    for k in sorted(tensors):
        if k.startswith("_"):
            continue
        h.update(k.encode())
        h.update(np.ascontiguousarray(tensors[k]).tobytes())
    return h.hexdigest()
