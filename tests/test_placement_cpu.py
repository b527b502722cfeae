"""Hot / cold placement (the gpu_idx / gpu_bucket contract) on CPU: exactness of the split solver against brute force, the
export rule of the reference (top-k by activation count, bucket sorted), whole-block buckets and multi-GPU dealing."""
import itertools
import os

import numpy as np
import pytest

from powerinfer_b200 import placement, synth


def brute_force(layer_counts, capacity, batch, threshold):
    pres = [np.concatenate([[0.0], np.cumsum(placement.layer_slice_values(c, batch))]) for c in layer_counts]
    cap, thr = capacity // batch, -(-threshold // batch) if threshold > 0 else 0
    best, best_ks = -1.0, None
    for ks in itertools.product(*[range(p.size) for p in pres]):
        if sum(ks) > cap or any(0 < k < thr for k in ks):
            continue
        v = sum(p[k] for p, k in zip(pres, ks))
        if v > best + 1e-9:
            best, best_ks = v, ks
    return best, best_ks


@pytest.mark.parametrize("seed", range(6))
def test_split_solver_is_optimal(seed):
    rng = np.random.default_rng(seed)
    L, F, batch = 4, 32, 4
    counts = [np.floor(rng.pareto(1.2, F) * 10) for _ in range(L)]
    for capacity, threshold in ((40, 0), (40, 12), (64, 8), (8, 12), (L * F, 0)):
        got = placement.solve_gpu_split(counts, capacity, batch, threshold)
        assert all(k % batch == 0 for k in got) and sum(got) <= capacity
        assert all(k == 0 or k >= threshold for k in got)
        best, _ = brute_force(counts, capacity, batch, threshold)
        mass = sum(np.sort(c)[::-1][:k].sum() for c, k in zip(counts, got))
        assert abs(mass - best) <= 1e-6 * max(1.0, best)


def test_whole_model_fits_means_everything_hot():
    counts = [np.arange(64.0) + 1, np.arange(64.0)[::-1] + 1]
    assert placement.solve_gpu_split(counts, 1 << 20, 8, 0) == [64, 64]
    assert placement.solve_gpu_split(counts, 0, 8, 0) == [0, 0]


def test_gpu_idx_and_bucket_follow_the_export_rule():
    rng = np.random.default_rng(1)
    counts = rng.permutation(256).astype(np.float64)                  # no ties: the top-k set is unique
    gpu_idx, bucket = placement.gpu_idx_and_bucket(counts, 40)
    assert gpu_idx.dtype == np.int32 and bucket.dtype == np.int32
    assert gpu_idx.sum() == 40 and np.all(np.diff(bucket) > 0)        # sorted global ids (export_split.py:40-41)
    assert set(bucket.tolist()) == set(np.argsort(-counts)[:40].tolist())
    assert np.array_equal(np.nonzero(gpu_idx)[0].astype(np.int32), bucket)
    assert counts[bucket].min() > counts[gpu_idx == 0].max()


def test_whole_block_bucket_and_dealing():
    F, mean = 4096, 0.1
    prof = synth.zipf_profile(F, mean)[np.random.default_rng(0).permutation(F)]
    gpu_idx, bucket = placement.bucket_of_whole_blocks(prof, 1024)
    assert bucket.size == 1024 and np.all(bucket.reshape(-1, 32)[:, 0] % 32 == 0)
    assert np.all(np.diff(bucket.reshape(-1, 32), axis=1) == 1)
    assert prof[bucket].sum() > 1024 / F * prof.sum()                 # hot blocks hold more than their share of the mass
    for n in (2, 4, 8):
        parts = placement.deal_across_gpus(prof, n)
        allids = np.sort(np.concatenate(parts))
        assert np.array_equal(allids, np.arange(F))                  # a partition
        masses = np.array([prof[p].sum() for p in parts])
        assert all(p.size == F // n and np.all(np.diff(p) > 0) for p in parts)
        assert masses.max() / masses.min() < 1.1                     # balanced expected active rows
    contiguous = np.array([np.sort(prof)[::-1][i * F // 4:(i + 1) * F // 4].sum() for i in range(4)])
    assert contiguous.max() / contiguous.min() > 3                    # what dealing avoids on a sorted profile


def test_vram_bytes():
    assert placement.vram_bytes([256, 512], 4608, 3) == 768 * 4608 * 3


def test_command_line_writes_the_gpu_index_file(tmp_path):
    """`python -m powerinfer_b200.placement` with powerinfer-py's flags: activation_<i>.pt files in, a PWRI GPU index file
    out whose tensors follow the export rule for the solver's per-layer counts (layer 10 must not sort before layer 2)."""
    import subprocess
    import sys
    import torch
    from powerinfer_b200 import gguf_loader, placement
    rng = np.random.default_rng(5)
    n_layer, F, batch = 12, 1024, 64
    counts = [np.floor(rng.pareto(1.2, F) * (1 + i)).astype(np.float32) for i in range(n_layer)]
    act = tmp_path / "act"
    act.mkdir()
    for i, c in enumerate(counts):
        torch.save(torch.from_numpy(c), act / f"activation_{i}.pt")
    out = tmp_path / "model.generated.gpuidx"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "powerinfer_b200.placement", "--activation", str(act), "--neuron", str(F),
                        "--capacity", str(3 * F), "--batch", str(batch), "--threshold", str(2 * batch),
                        "--vram-capacity", str(123456789), "--output", str(out)], capture_output=True, text=True, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    idx, bucket, vram = gguf_loader.load_gpu_split(str(out))
    assert vram == 123456789 and len(idx) == n_layer
    solved = placement.solve_gpu_split(counts, 3 * F, batch, 2 * batch)
    assert sum(solved) <= 3 * F and all(k == 0 or k >= 2 * batch for k in solved)
    for i in range(n_layer):
        want_idx, want_bucket = placement.gpu_idx_and_bucket(counts[i], solved[i])
        assert np.array_equal(idx[i], want_idx) and np.array_equal(bucket[i], want_bucket)
        assert len(bucket[i]) == solved[i] and np.all(np.diff(bucket[i]) > 0)
    # a wrong --neuron is refused
    r = subprocess.run([sys.executable, "-m", "powerinfer_b200.placement", "--activation", str(act), "--neuron", str(F + 64),
                        "--output", str(out)], capture_output=True, text=True, cwd=root)
    assert r.returncode != 0 and "counts" in r.stderr
