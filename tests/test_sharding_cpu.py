"""The N > 1 host logic on CPU: two gloo ranks each take their slice of one layer, compute their partial d_model
vectors with the CPU checker, all-reduce them, and must reproduce the unsharded operators.

Checks the two facts the sharded engine relies on: (1) whole heads / whole 32-neuron blocks per rank leave every
quantised activation block and every axpy coefficient unchanged, so the only difference to the single-GPU result is the
order of FP32 additions; (2) the exchange is a plain sum over ranks of the out-projection and down-projection partials.
"""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from powerinfer_b200 import sharding, synth  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, wtype, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import pio
    o = pio.Oracle()
    spec = synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=wtype, n_layer=1, d=512, n_ff=2048, n_head=4, n_head_kv=2, rank=64,
                           firing=0.2, seed=77)
    t = synth.build_model(spec)
    sl = sharding.shard_layer(spec, t, 0, world, rank)
    rng = np.random.default_rng(5)                       # same draw on every rank
    d, F, hd = spec.d, spec.n_ff, spec.head_dim
    x = rng.standard_normal((1, d), dtype=np.float32)
    att = rng.standard_normal((1, d), dtype=np.float32)
    dq, Fl = d // world, F // world
    # --- attention out-projection: columns of this rank's heads
    part = o.mul_mat(wtype, np.ascontiguousarray(sl["wo"]), d, dq, att[:, rank * dq:(rank + 1) * dq])
    tot = torch.from_numpy(part.copy())
    dist.all_reduce(tot)
    full = o.mul_mat(wtype, t["blk.0.attn_output.weight"], d, d, att)
    err_wo = float(np.abs(tot.numpy() - full).max())
    # --- qkv rows: this rank's q heads, k heads, v heads
    qkv = o.mul_mat(wtype, np.ascontiguousarray(sl["wqkv"]), sl["wqkv"].shape[0], d, x)
    q_full = o.mul_mat(wtype, t["blk.0.attn_q.weight"], d, d, x)
    k_full = o.mul_mat(wtype, t["blk.0.attn_k.weight"], spec.d_kv, d, x)
    dkvl = spec.d_kv // world
    ok_qkv = (np.array_equal(qkv[:, :dq], q_full[:, rank * dq:(rank + 1) * dq])
              and np.array_equal(qkv[:, dq:dq + dkvl], k_full[:, rank * dkvl:(rank + 1) * dkvl]))
    # --- sparse FFN on this rank's neurons: predictor slice, up/gate, axpy partial
    hid = np.maximum(o.mul_mat(synth.F16, t["blk.0.fc1.weight"], spec.rank, d, x), 0)
    pred_full = o.mul_mat(synth.F16, t["blk.0.fc2.weight"], F, spec.rank, hid)
    pred = o.mul_mat(synth.F16, np.ascontiguousarray(sl["fc2"]), Fl, spec.rank, hid)
    ok_pred = np.array_equal(pred, pred_full[:, rank * Fl:(rank + 1) * Fl])
    up = o.mul_mat_idx(wtype, np.ascontiguousarray(sl["up"]), Fl, d, x, pred)
    gate = o.mul_mat_idx(wtype, np.ascontiguousarray(sl["gate"]), Fl, d, x, pred)
    h = np.maximum(gate, 0) * up
    part = o.axpy(wtype, np.ascontiguousarray(sl["down_t"]), Fl, d, h, pred, np.zeros(Fl, np.int32))
    tot2 = torch.from_numpy(part.copy())
    dist.all_reduce(tot2)
    up_f = o.mul_mat_idx(wtype, t["blk.0.ffn_up.weight"], F, d, x, pred_full)
    gate_f = o.mul_mat_idx(wtype, t["blk.0.ffn_gate.weight"], F, d, x, pred_full)
    h_f = np.maximum(gate_f, 0) * up_f
    full2 = o.axpy(wtype, t["blk.0.ffn_down_t.weight"], F, d, h_f, pred_full, np.zeros(F, np.int32))
    err_ffn = float(np.abs(tot2.numpy() - full2).max())
    n_active = torch.tensor([int((pred >= 0).sum())])
    dist.all_reduce(n_active)
    np.save(os.path.join(out_dir, f"r{rank}.npy"),
            np.array([err_wo, err_ffn, float(ok_qkv), float(ok_pred), float(n_active.item()), float((pred_full >= 0).sum())]))
    dist.destroy_process_group()


@pytest.mark.parametrize("wtype", [synth.F16, synth.Q4_0])
def test_two_ranks_reproduce_the_unsharded_layer(tmp_path, wtype):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), wtype, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err_wo, err_ffn, ok_qkv, ok_pred, n_act, n_act_full = np.load(tmp_path / f"r{r}.npy")
        assert ok_qkv == 1.0 and ok_pred == 1.0
        assert n_act == n_act_full                     # the ranks' active sets partition the global one
        assert err_wo <= 1e-5 and err_ffn <= 1e-5, (err_wo, err_ffn)


def test_shard_shapes_and_block_alignment():
    spec = synth.ModelSpec(arch=synth.ARCH_FALCON, wtype=synth.Q4_0, n_layer=1, d=512, n_ff=2048, n_head=8, n_head_kv=2, rank=64)
    t = synth.build_model(spec)
    for world in (1, 2):
        rows = 0
        for r in range(world):
            sl = sharding.shard_layer(spec, t, 0, world, r)
            dq, dkv = spec.d // world, spec.d_kv // world
            assert sl["wqkv"].shape == (dq + 2 * dkv, spec.d // 32 * 18)
            assert sl["wo"].shape == (spec.d, dq // 32 * 18)
            assert sl["up"].shape[0] == spec.n_ff // world and sl["up"].shape[0] % 32 == 0
            assert sl["gate"] is None and sl["fc2"].shape == (spec.n_ff // world, spec.rank)
            rows += sl["down_t"].shape[0]
        assert rows == spec.n_ff


def test_eight_rank_shards_partition_heads_and_neurons():
    """The 8-GPU split of a model with the headline's proportions (8 heads and one KV head per rank, neurons in whole
    32-blocks): shapes per rank, and the ranks' rows put together give back the unsharded tensors."""
    spec = synth.ModelSpec(arch=synth.ARCH_LLAMA, wtype=synth.F16, n_layer=1, d=1024, n_ff=4096, n_head=64, n_head_kv=8, rank=64)
    t = synth.build_model(spec)
    world = 8
    full = sharding.shard_layer(spec, t, 0, 1, 0)
    ups, downs, fc2s = [], [], []
    for r in range(world):
        sl = sharding.shard_layer(spec, t, 0, world, r)
        dq, dkv = spec.d // world, spec.d_kv // world
        assert sl["wqkv"].shape[0] == dq + 2 * dkv and dkv == spec.d_kv // spec.n_head_kv      # exactly one KV head
        assert sl["wo"].shape[0] == spec.d
        assert sl["up"].shape[0] == spec.n_ff // world and sl["up"].shape[0] % 32 == 0
        assert np.array_equal(sl["fc1"], full["fc1"])                                           # replicated
        ups.append(sl["up"]); downs.append(sl["down_t"]); fc2s.append(sl["fc2"])
    assert np.array_equal(np.concatenate(ups), full["up"])
    assert np.array_equal(np.concatenate(downs), full["down_t"])
    assert np.array_equal(np.concatenate(fc2s), full["fc2"])
