"""Argument validation of the C ABI happens before any CUDA call, so it can be held to its contract without a device:
bad shapes, null or misaligned pointers and undersized workspaces come back as PI_ERR_INVALID (1) / PI_ERR_WORKSPACE (3)
with a message, for every operator entry point and for the engine's configuration."""
import ctypes as C

import pytest

from powerinfer_b200 import _lib
from powerinfer_b200.engine import EngineConfig, lib as elib

lib = _lib.lib
F16, Q4 = _lib.PI_TYPE_F16, _lib.PI_TYPE_Q4_0
P = 1 << 20                      # a fake, suitably aligned "device pointer": validation never dereferences it
WS, WSN = 1 << 21, 1 << 26       # fake workspace pointer (256-aligned) and a generous size
INVALID, WORKSPACE = 1, 3


def err():
    return lib.pi_last_error().decode()


@pytest.mark.parametrize("call,code,needle", [
    (lambda: lib.pi_mul_mat(7, P, 8, 256, P, 1, None, P, WS, WSN, None), INVALID, "unknown weight type"),
    (lambda: lib.pi_mul_mat(Q4, P, 8, 100, P, 1, None, P, WS, WSN, None), INVALID, "256"),
    (lambda: lib.pi_mul_mat(F16, P, 8, 12, P, 1, None, P, WS, WSN, None), INVALID, "% 8"),
    (lambda: lib.pi_mul_mat(F16, P + 2, 8, 256, P, 1, None, P, WS, WSN, None), INVALID, "16-byte aligned"),
    (lambda: lib.pi_mul_mat(F16, None, 8, 256, P, 1, None, P, WS, WSN, None), INVALID, "non-null"),
    (lambda: lib.pi_mul_mat(F16, P, 8, 256, None, 1, None, P, WS, WSN, None), INVALID, "mul_mat"),
    (lambda: lib.pi_mul_mat(F16, P, 8, 256, P, 1, None, P, WS + 8, WSN, None), WORKSPACE, "workspace"),
    (lambda: lib.pi_mul_mat(F16, P, 8, 256, P, 4, None, P, WS, 64, None), WORKSPACE, "workspace"),
    (lambda: lib.pi_mul_mat_idx(F16, P, 64, 256, P, 1, P, 64, None, 0.0, P, 32, WS, WSN, None), INVALID, "n_w_rows"),
    (lambda: lib.pi_mul_mat_idx(F16, P, 32, 256, P, 1, P, 64, None, 0.0, P, 64, WS, WSN, None), INVALID, "bucket"),
    (lambda: lib.pi_mul_mat_idx(F16, P, 64, 256, P, 1, P, 32, None, 0.0, P, 64, WS, WSN, None), INVALID, "idx_stride"),
    (lambda: lib.pi_mul_mat_idx(F16, P, 64, 256, P, 1, P, 64, None, 0.0, P, 64, WS, 128, None), WORKSPACE, "workspace"),
    (lambda: lib.pi_axpy(Q4, P, 64, 256, P, 1, 70, P, 70, None, 0.0, P, WS, WSN, None), INVALID, "h_stride"),
    (lambda: lib.pi_axpy(F16, P, 64, 256, P, 1, 32, P, 64, None, 0.0, P, WS, WSN, None), INVALID, "axpy"),
    (lambda: lib.pi_axpy(F16, P, 64, 256, P, 1, 64, P, 64, None, 0.0, P, WS, 128, None), WORKSPACE, "workspace"),
    (lambda: lib.pi_sparse_ffn(F16, P, None, None, 64, 256, P, 1, P, 64, None, 0.0, None, P, WS, WSN, None), INVALID, "sparse_ffn"),
    (lambda: lib.pi_sparse_ffn(Q4, P, P, P, 64, 256, P, 1, P, 72, None, 0.0, None, P, WS, WSN, None), INVALID, "% 32"),
    (lambda: lib.pi_predictor(P, P, 250, 64, 128, P, 1, P, WS, WSN, None), INVALID, "% 8"),
    (lambda: lib.pi_active_list(P, 64, 0, 64, 0.0, P, P, WS, WSN, None), INVALID, "active_list"),
    (lambda: lib.pi_active_list(P, 64, 1, 32, 0.0, P, P, WS, WSN, None), INVALID, "active_list"),
    (lambda: lib.pi_norm(P + 4, 1, 256, 1, 1e-5, None, None, P, None), INVALID, "16-byte aligned"),
    (lambda: lib.pi_rope(P, 1, 4, 63, P, P, 0, None), INVALID, "rope"),
    (lambda: lib.pi_quantize_q4_0(P, P, 4, 100, None), INVALID, "quantize_q4_0"),
    (lambda: lib.pi_q4_0_repack(P, P, 4, 256, None), INVALID, "q4_0_repack"),
    (lambda: lib.pi_q4_0_repack(P, P + 8, 4, 256, None), INVALID, "16-byte aligned"),
    (lambda: lib.pi_axpy_static(F16, P, 1 << 17, 256, P, 1 << 17, P, 1 << 17, None, 0.0, P, None), INVALID, "pi_axpy"),
])
def test_bad_arguments_are_refused_before_any_launch(call, code, needle):
    rc = call()
    assert rc == code, (rc, err())
    assert needle in err(), err()


def test_zero_work_is_ok_without_a_device():
    assert lib.pi_mul_mat(F16, P, 8, 256, P, 0, None, P, WS, WSN, None) == 0          # no tokens
    assert lib.pi_mul_mat(F16, P, 0, 256, P, 1, None, P, WS, WSN, None) == 0          # no rows
    assert lib.pi_mul_mat_idx(F16, P, 0, 256, P, 0, P, 0, None, 0.0, P, 0, WS, WSN, None) == 0
    assert lib.pi_axpy(F16, P, 64, 256, P, 0, 64, P, 64, None, 0.0, P, WS, WSN, None) == 0


def good_config(**over):
    c = dict(arch=0, wtype=F16, n_layer=2, d=256, n_ff=1280, n_head=4, n_head_kv=4, rank=64, n_vocab=512, n_ctx=128, n_pos=0,
             norm_eps=1e-5, rope_base=10000.0, threshold=0.0, max_batch=1, n_ranks=1, rank_id=0)
    c.update(over)
    return EngineConfig(**c)


@pytest.mark.parametrize("over,needle", [
    (dict(arch=9), "unknown arch"), (dict(wtype=5), "unknown weight type"), (dict(n_layer=0), "non-positive"),
    (dict(n_head=3), "n_head"), (dict(n_head_kv=3), "n_head_kv"), (dict(max_batch=33), "max_batch"),
    (dict(n_ranks=2, rank_id=2), "bad rank"), (dict(n_ff=1296), "32 x n_ranks"), (dict(n_ranks=8), "n_head_kv"),
    (dict(d=320, n_head=4), "head_dim"), (dict(wtype=Q4, d=128, n_head=4), "multiples of 256"), (dict(rank=60), "rank"),
])
def test_engine_configurations_are_validated(over, needle):
    cfg = good_config(**over)
    assert elib.pi_engine_workspace_bytes(C.byref(cfg)) == 0
    assert needle in err(), err()


def test_engine_sizes_for_good_configurations():
    for over in (dict(), dict(arch=3), dict(arch=1, n_head_kv=2), dict(arch=2, n_pos=2050), dict(wtype=Q4), dict(max_batch=8),
                 dict(n_ranks=2, rank_id=1)):
        cfg = good_config(**over)
        assert elib.pi_engine_workspace_bytes(C.byref(cfg)) > 0, err()
        assert elib.pi_engine_kv_bytes(C.byref(cfg)) == 2 * cfg.max_batch * 128 * (256 // 4 * cfg.n_head_kv // cfg.n_ranks) * 2
