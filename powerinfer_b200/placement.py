"""Hot / cold neuron placement: which FFN neurons' rows are resident in which memory.

The reference decides this offline (powerinfer-py/powerinfer/solver.py:10-90, export_split.py:24-76) and at load time
(llama.cpp:2781-2997): per layer, the k neurons with the highest profiled activation counts go to the GPU; k per layer
comes from an integer program that maximises the covered activation mass under a VRAM cap, in slices of `batch` neurons,
where a layer gets either nothing or at least `threshold` neurons.  The result travels as two int32 tensors per layer:
`gpu_idx[F]` (1 = row lives on the GPU; the CPU operator skips it, ggml.c:14211) and `gpu_bucket[k]` = the SORTED
global ids of the GPU rows (the GPU operator maps local row r to neuron gpu_bucket[r], ggml-cuda.cu:4694).

Here the same contract is produced without an external solver: within a layer the slices are sorted by count, so a layer's
choice is a prefix length, the objective is separable, and the optimum is a max-plus convolution over the layers (exact,
O(layers x capacity x slices)).  `deal_across_gpus` is the multi-GPU analogue: whole 32-neuron blocks dealt round-robin in
descending order of firing mass, so every GPU expects the same number of active rows under a power-law profile.
"""
from __future__ import annotations

import numpy as np


def layer_slice_values(counts: np.ndarray, batch: int) -> np.ndarray:
    """Activation mass of each slice of `batch` neurons of one layer, neurons sorted by count, descending
    (solver.py:21-27).  The neuron count must be a multiple of `batch`, as the reference's view(-1, batch) requires."""
    c = np.sort(np.asarray(counts, dtype=np.float64))[::-1]
    if c.size % batch != 0:
        raise ValueError(f"{c.size} neurons are not a multiple of the slice size {batch}")
    return c.reshape(-1, batch).sum(axis=1)


def solve_gpu_split(layer_counts: list, capacity: int, batch: int = 256, threshold: int = 0) -> list:
    """Neurons to place on the GPU per layer (multiples of `batch`), maximising the sum of their activation counts with
    at most `capacity` neurons in total; a layer gets 0 or at least `threshold` neurons (solver.py:36-68).

    Exact: dp[c] = best mass with c slices over the layers seen so far; a layer contributes its prefix sums."""
    cap = int(capacity // batch)
    thr = int(-(-threshold // batch)) if threshold > 0 else 0          # slices; a positive threshold rounds up
    prefixes = []
    for counts in layer_counts:
        v = layer_slice_values(counts, batch)
        prefixes.append(np.concatenate([[0.0], np.cumsum(v)]))
    neg = -np.inf
    dp = np.full(cap + 1, neg)
    dp[0] = 0.0
    choice = []
    for pre in prefixes:
        n = pre.size - 1
        new = dp.copy()                                                  # k = 0
        arg = np.zeros(cap + 1, dtype=np.int64)
        for k in range(max(thr, 1), min(n, cap) + 1):
            cand = np.full(cap + 1, neg)
            cand[k:] = dp[: cap + 1 - k] + pre[k]
            better = cand > new                                          # ties keep the smaller k
            new[better] = cand[better]
            arg[better] = k
        choice.append(arg)
        dp = new
    c = int(np.argmax(dp))                                               # smallest capacity reaching the best mass
    ks = []
    for arg in reversed(choice):
        k = int(arg[c])
        ks.append(k)
        c -= k
    return [k * batch for k in reversed(ks)]


def gpu_idx_and_bucket(counts: np.ndarray, k: int):
    """The two tensors export_split.py:24-52 writes for one layer: top-k neurons by count -> gpu_idx (0/1 int32 [F]) and
    gpu_bucket (their ids, ascending).  Ties go to the lower id (the reference's torch.topk leaves ties unspecified)."""
    counts = np.asarray(counts)
    order = np.argsort(-counts.astype(np.float64), kind="stable")
    hot = np.sort(order[: int(k)]).astype(np.int32)
    gpu_idx = np.zeros(counts.size, dtype=np.int32)
    gpu_idx[hot] = 1
    return gpu_idx, hot


def bucket_of_whole_blocks(counts: np.ndarray, k: int, block: int = 32):
    """Like gpu_idx_and_bucket, but the unit is a block of `block` consecutive neurons (ranked by the block's total count):
    the Q4_0 axpy quantises the hidden vector per 32 consecutive neurons (ggml.c:14465-14618), so a device must hold whole
    blocks for its coefficients to equal the single-device ones."""
    counts = np.asarray(counts, dtype=np.float64)
    if counts.size % block != 0 or k % block != 0:
        raise ValueError("neuron count and k must be multiples of the block size")
    mass = counts.reshape(-1, block).sum(axis=1)
    order = np.argsort(-mass, kind="stable")[: k // block]
    blocks = np.sort(order)
    hot = (blocks[:, None] * block + np.arange(block)[None, :]).reshape(-1).astype(np.int32)
    gpu_idx = np.zeros(counts.size, dtype=np.int32)
    gpu_idx[hot] = 1
    return gpu_idx, hot


def deal_across_gpus(counts: np.ndarray, n_gpus: int, block: int = 32) -> list:
    """Sorted global ids per GPU: blocks of `block` neurons dealt round-robin (boustrophedon) in descending order of
    firing mass, so the expected number of active rows is the same on every GPU; every neuron lands on exactly one GPU."""
    counts = np.asarray(counts, dtype=np.float64)
    if counts.size % block != 0:
        raise ValueError("neuron count must be a multiple of the block size")
    mass = counts.reshape(-1, block).sum(axis=1)
    order = np.argsort(-mass, kind="stable")
    owner = np.empty(order.size, dtype=np.int64)
    pos = np.arange(order.size)
    rnd, slot = pos // n_gpus, pos % n_gpus
    owner[order] = np.where(rnd % 2 == 0, slot, n_gpus - 1 - slot)      # 0..n-1, n-1..0, 0..n-1: evens out the rank bias
    out = []
    for g in range(n_gpus):
        blocks = np.sort(np.nonzero(owner == g)[0])
        out.append((blocks[:, None] * block + np.arange(block)[None, :]).reshape(-1).astype(np.int32))
    return out


def vram_bytes(neurons_per_layer: list, row_bytes: int, n_mats: int) -> int:
    """Bytes of FFN rows the placement keeps on the GPU: n_mats rows (gate, up, down_t) of row_bytes per hot neuron."""
    return int(sum(neurons_per_layer)) * row_bytes * n_mats


def load_activation_counts(directory: str) -> list:
    """`activation_<i>.pt` files of a profiling run (one 1-D tensor of per-neuron activation counts per layer), in layer
    order, as float64 arrays.  The reference sorts the file names as strings (export_split.py:16-22), which puts
    activation_10 before activation_2; here they are ordered by layer number, which is what the solver's
    `activation_{i}.pt` loop (solver.py:20-22) reads."""
    import os
    import re
    import torch
    found = {}
    for f in os.listdir(directory):
        m = re.fullmatch(r"activation_(\d+)\.pt", f)
        if m:
            found[int(m.group(1))] = os.path.join(directory, f)
    if not found or sorted(found) != list(range(len(found))):
        raise ValueError(f"{directory}: expected activation_0.pt .. activation_<n-1>.pt, found layers {sorted(found)}")
    return [torch.load(found[i], map_location="cpu").to(torch.float64).reshape(-1).numpy() for i in range(len(found))]


def main(argv=None) -> int:
    """`python -m powerinfer_b200.placement`: the command line of powerinfer-py (`python -m powerinfer`, __main__.py:10-46)
    with the same flags: profile directory -> per-layer neuron counts under the capacity -> `.generated.gpuidx` file."""
    import argparse
    from . import gguf_loader
    ap = argparse.ArgumentParser(prog="python -m powerinfer_b200.placement",
                                 description="Choose the GPU-resident FFN neurons of every layer under a capacity and write the GPU index file.")
    ap.add_argument("--activation", required=True, help="directory with activation_<layer>.pt count tensors")
    ap.add_argument("--neuron", type=int, default=8192 * 4, help="neurons per layer")
    ap.add_argument("--capacity", type=int, default=int(8192 * 4 * 32 * 0.1), help="neurons that fit on the GPU in total")
    ap.add_argument("--layer", type=int, default=None, help="layers to place (default: every activation file)")
    ap.add_argument("--vram-capacity", type=int, default=0, help="bytes of VRAM the split was made for (recorded in the file)")
    ap.add_argument("--batch", type=int, default=256, help="neurons per placement slice")
    ap.add_argument("--threshold", type=int, default=0, help="a layer gets no neurons or at least this many")
    ap.add_argument("--whole-blocks", action="store_true", help="place whole blocks of 32 consecutive neurons (needed for a Q4_0 down_t bucket)")
    ap.add_argument("--output", required=True, help="path of the GPU index file to write")
    a = ap.parse_args(argv)
    counts = load_activation_counts(a.activation)
    if a.layer is not None:
        if a.layer > len(counts):
            raise SystemExit(f"--layer {a.layer} but only {len(counts)} activation files")
        counts = counts[: a.layer]
    for i, c in enumerate(counts):
        if c.size != a.neuron:
            raise SystemExit(f"layer {i}: {c.size} counts, --neuron says {a.neuron}")
    solved = solve_gpu_split(counts, a.capacity, a.batch, a.threshold)
    pick = bucket_of_whole_blocks if a.whole_blocks else gpu_idx_and_bucket
    idx, bucket = zip(*(pick(c, k) for c, k in zip(counts, solved)))
    gguf_loader.write_gpu_split(a.output, list(idx), list(bucket), a.vram_capacity)
    print(f"solved: {solved}, total neurons: {sum(solved)}")
    print(f"exported GPU index to {a.output}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
