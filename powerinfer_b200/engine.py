"""Host-side driver of the decode engine: weight upload / sharding, buffers, and the llama_decode-style step.

Mirrors the reference's calling sequence (llama.h): build a model once (llama_load_model_from_file +
llama_new_context_with_model), then `decode(tokens, pos)` per step (llama_decode) and read `logits`
(llama_get_logits) or the greedy ids (llama_sample_token_greedy).  All compute happens in
libpowerinfer_b200.so; torch provides device memory, streams and (for sharded runs) the process group used
to hand IPC handles around.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import synth
from ._lib import PI_TYPE_F16, PI_TYPE_Q4_0, check, lib

PI_MAX_RANKS = 8
PI_ARCH_BAMBOO = 3                     # the llama graph with the symmetric gate relu(gate) * relu(up)
N_STAGES = 12
STAGE_NAMES = ["norm", "qkv", "attention", "out_proj", "predictor", "compact", "up_gate", "down", "lm_head", "exchange", "other", "sparse_ffn"]

_vp = C.c_void_p


class EngineConfig(C.Structure):
    _fields_ = [("arch", C.c_int), ("wtype", C.c_int), ("n_layer", C.c_int), ("d", C.c_int), ("n_ff", C.c_int),
                ("n_head", C.c_int), ("n_head_kv", C.c_int), ("rank", C.c_int), ("n_vocab", C.c_int), ("n_ctx", C.c_int),
                ("n_pos", C.c_int), ("norm_eps", C.c_float), ("rope_base", C.c_float), ("threshold", C.c_float),
                ("max_batch", C.c_int), ("n_ranks", C.c_int), ("rank_id", C.c_int)]


class LayerWeights(C.Structure):
    _fields_ = [(n, _vp) for n in ("attn_norm_w", "attn_norm_b", "attn_norm2_w", "attn_norm2_b", "wqkv", "bqkv", "wo", "bo",
                                   "ffn_norm_w", "ffn_norm_b", "fc1", "fc2", "gate", "up", "down_t", "up_b", "down_b")]


class ModelWeights(C.Structure):
    _fields_ = [(n, _vp) for n in ("tok_embd", "pos_embd", "out_norm_w", "out_norm_b", "output")]


class Exchange(C.Structure):
    _fields_ = [("n_ranks", C.c_int), ("rank_id", C.c_int), ("slot_floats", C.c_int64),
                ("mailbox_local", _vp), ("mailbox_peer", _vp * PI_MAX_RANKS), ("epoch", _vp)]


for _name, _res, _args in [
    ("pi_engine_workspace_bytes", C.c_size_t, [C.POINTER(EngineConfig)]),
    ("pi_engine_kv_bytes", C.c_size_t, [C.POINTER(EngineConfig)]),
    ("pi_engine_create", C.c_int, [C.POINTER(EngineConfig), C.POINTER(ModelWeights), C.POINTER(LayerWeights), _vp, C.c_size_t,
                                   _vp, _vp, _vp, C.POINTER(_vp)]),
    ("pi_engine_destroy", None, [_vp]),
    ("pi_engine_set_exchange", C.c_int, [_vp, C.POINTER(Exchange)]),
    ("pi_engine_io", C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp)]),
    ("pi_engine_decode", C.c_int, [_vp, C.c_int, _vp]),
    ("pi_engine_advance", C.c_int, [_vp, C.c_int, _vp]),
    ("pi_engine_decode_host", C.c_int, [_vp, _vp, _vp, C.c_int, _vp, _vp, _vp]),
    ("pi_engine_prefill_host", C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    ("pi_engine_profile_step", C.c_int, [_vp, C.c_int, _vp, C.POINTER(C.c_int), _vp]),
    ("pi_engine_status", C.c_int, [_vp, _vp]),
    ("pi_engine_set_wait_cycles", C.c_int, [_vp, C.c_longlong]),
    ("pi_engine_debug", C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp)]),
    ("pi_engine_launches", C.c_int, [_vp]),
    ("pi_engine_set_trace", C.c_int, [_vp, _vp]),
    ("pi_engine_active_total", C.c_int, [_vp, C.c_int, C.POINTER(C.c_uint64), _vp]),
    ("pi_device_malloc", C.c_int, [C.POINTER(_vp), C.c_size_t]),
    ("pi_device_free", C.c_int, [_vp]),
    ("pi_ipc_export", C.c_int, [_vp, _vp]),
    ("pi_ipc_import", C.c_int, [_vp, C.POINTER(_vp)]),
    ("pi_ipc_close", C.c_int, [_vp]),
    ("pi_engine_time_stage", C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int), _vp]),
]:
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args

ENGINE_EXPORTS = ["pi_engine_workspace_bytes", "pi_engine_kv_bytes", "pi_engine_create", "pi_engine_destroy",
                  "pi_engine_set_exchange", "pi_engine_io", "pi_engine_decode", "pi_engine_advance", "pi_engine_decode_host", "pi_engine_prefill_host",
                  "pi_engine_profile_step", "pi_engine_time_stage", "pi_engine_status", "pi_engine_set_wait_cycles", "pi_engine_debug", "pi_engine_launches", "pi_engine_set_trace", "pi_engine_active_total",
                  "pi_device_malloc", "pi_device_free", "pi_ipc_export", "pi_ipc_import", "pi_ipc_close"]


from .sharding import shard_cols, shard_layer, shard_rows  # noqa: E402,F401  (host-only logic, importable without the CUDA library)


# ------------------------------------------------------------------------------------------------ device side

def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        a = torch.from_numpy(np.ascontiguousarray(a))
    return a.contiguous().cuda()


def _upload2d(a, wtype: int):
    """F16 [rows, cols] stays as is; Q4_0 ggml block bytes [rows, cols/32*18] are re-laid out (pi_q4_0_repack)."""
    a = _dev(a)
    if a.dtype == torch.float16:
        return a
    assert a.dtype == torch.uint8 and wtype == PI_TYPE_Q4_0
    rows, ncols = a.shape[0], a.shape[1] // 18 * 32
    out = torch.empty_like(a)
    check(lib.pi_q4_0_repack(a.data_ptr(), out.data_ptr(), rows, ncols, _stream()))
    return out


def _ptr(t):
    return None if t is None else t.data_ptr()


class DecodeEngine:
    """One rank of the decode loop.  `tensors` holds the FULL model under the reference's GGUF tensor names (numpy or
    torch); this rank uploads its slice."""

    def __init__(self, spec: synth.ModelSpec, tensors: dict, max_batch: int = 1, n_ranks: int = 1, rank: int = 0,
                 local_layers: list | None = None):
        self.spec, self.max_batch, self.n_ranks, self.rank = spec, max_batch, n_ranks, rank
        n_pos = synth.OPT_N_POS if spec.arch == synth.ARCH_OPT else 0
        self.cfg = EngineConfig(PI_ARCH_BAMBOO if getattr(spec, "gate_sym", False) else spec.arch, spec.wtype, spec.n_layer, spec.d, spec.n_ff, spec.n_head, spec.n_head_kv, spec.rank,
                                spec.n_vocab, spec.n_ctx, n_pos, spec.norm_eps, spec.rope_base, spec.threshold, max_batch,
                                n_ranks, rank)
        ws_bytes = lib.pi_engine_workspace_bytes(C.byref(self.cfg))
        if ws_bytes == 0:
            check(1)
        self.keep = []                       # device tensors the engine points into

        def hold(x):
            if x is not None:
                self.keep.append(x)
            return x

        self.layers = (LayerWeights * spec.n_layer)()
        for il in range(spec.n_layer):
            sl = local_layers[il] if local_layers is not None else shard_layer(spec, tensors, il, n_ranks, rank)
            L = self.layers[il]
            for name in ("attn_norm.weight", "attn_norm.bias", "attn_norm_2.weight", "attn_norm_2.bias", "ffn_norm.weight", "ffn_norm.bias"):
                field = {"attn_norm.weight": "attn_norm_w", "attn_norm.bias": "attn_norm_b", "attn_norm_2.weight": "attn_norm2_w",
                         "attn_norm_2.bias": "attn_norm2_b", "ffn_norm.weight": "ffn_norm_w", "ffn_norm.bias": "ffn_norm_b"}[name]
                setattr(L, field, _ptr(hold(_dev(sl.get(name)))))
            for name in ("wqkv", "wo", "gate", "up", "down_t"):
                a = sl.get(name)
                setattr(L, name, _ptr(hold(None if a is None else _upload2d(a, spec.wtype))))
            for name in ("fc1", "fc2"):
                setattr(L, name, _ptr(hold(_dev(sl[name]))))
            for name in ("bqkv", "bo", "up_b", "down_b"):
                setattr(L, name, _ptr(hold(_dev(sl.get(name)))))
        g = tensors
        self.globals = ModelWeights(
            _ptr(hold(_dev(g["token_embd.weight"]))), _ptr(hold(_dev(g.get("position_embd.weight")))),
            _ptr(hold(_dev(g["output_norm.weight"]))), _ptr(hold(_dev(g.get("output_norm.bias")))),
            _ptr(hold(None if g.get("output.weight") is None else _upload2d(g["output.weight"], spec.wtype))))
        kv_bytes = lib.pi_engine_kv_bytes(C.byref(self.cfg))
        self.k_cache = torch.zeros(kv_bytes // 2, dtype=torch.float16, device="cuda")
        self.v_cache = torch.zeros(kv_bytes // 2, dtype=torch.float16, device="cuda")
        self.ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device="cuda")
        off = (-self.ws.data_ptr()) % 256
        self.handle = _vp()
        # the step is captured into a CUDA graph, which the legacy default stream cannot do: the engine owns a stream
        self.stream = torch.cuda.Stream()
        self.st = self.stream.cuda_stream
        torch.cuda.synchronize()
        check(lib.pi_engine_create(C.byref(self.cfg), C.byref(self.globals), self.layers, self.ws.data_ptr() + off, ws_bytes,
                                   self.k_cache.data_ptr(), self.v_cache.data_ptr(), self.st, C.byref(self.handle)))
        tok, pos, logits, amax = _vp(), _vp(), _vp(), _vp()
        check(lib.pi_engine_io(self.handle, C.byref(tok), C.byref(pos), C.byref(logits), C.byref(amax)))
        self.io = (tok.value, pos.value, logits.value, amax.value)
        # pinned host staging for the host-buffer entry point
        self.h_tokens = torch.zeros(max_batch, dtype=torch.int32).pin_memory()
        self.h_pos = torch.zeros(max_batch, dtype=torch.int32).pin_memory()
        self.h_logits = torch.zeros(max_batch, spec.n_vocab, dtype=torch.float32).pin_memory()
        self.h_argmax = torch.zeros(max_batch, dtype=torch.int32).pin_memory()
        self._xch_mem = None

    # ---- llama_decode + llama_get_logits with host buffers
    def decode(self, tokens, pos, want_logits: bool = True):
        T = len(tokens)
        self.h_tokens[:T] = torch.as_tensor(tokens, dtype=torch.int32)
        self.h_pos[:T] = torch.as_tensor(pos, dtype=torch.int32)
        check(lib.pi_engine_decode_host(self.handle, self.h_tokens.data_ptr(), self.h_pos.data_ptr(), T,
                                        self.h_logits.data_ptr() if want_logits else None, self.h_argmax.data_ptr(), self.st))
        return (self.h_logits[:T].numpy() if want_logits else None), self.h_argmax[:T].numpy()

    def prefill(self, tokens, seq: int = 0, pos0: int = 0, want_logits: bool = True):
        """Prompt processing: `tokens` are consecutive tokens of sequence `seq` starting at position pos0; they go through
        in chunks of up to max_batch tokens per step.  Returns (logits of the last token | None, its greedy id | None)."""
        toks = np.ascontiguousarray(np.asarray(tokens, np.int32))
        logits = np.empty(self.spec.n_vocab, np.float32) if want_logits else None
        amax = np.zeros(1, np.int32)
        check(lib.pi_engine_prefill_host(self.handle, toks.ctypes.data, len(toks), seq, pos0,
                                         logits.ctypes.data if want_logits else None, amax.ctypes.data if want_logits else None, self.st))
        return logits, (int(amax[0]) if want_logits else None)

    def decode_host_raw(self, T: int, want_logits: bool = True):
        """The same call with the staging buffers already filled (benchmark inner loop: no Python-side copies)."""
        check(lib.pi_engine_decode_host(self.handle, self.h_tokens.data_ptr(), self.h_pos.data_ptr(), T,
                                        self.h_logits.data_ptr() if want_logits else None, self.h_argmax.data_ptr(), self.st))

    # ---- device-resident step: inputs already in the engine's device buffers
    def set_inputs_device(self, tokens, pos):
        T = len(tokens)
        self.h_tokens[:T] = torch.as_tensor(tokens, dtype=torch.int32)
        self.h_pos[:T] = torch.as_tensor(pos, dtype=torch.int32)
        with torch.cuda.stream(self.stream):
            self.device_view("tokens", T).copy_(self.h_tokens[:T], non_blocking=True)
            self.device_view("pos", T).copy_(self.h_pos[:T], non_blocking=True)
        self.stream.synchronize()            # the pinned staging buffers are reused by the next call

    def step_device(self, T: int):
        check(lib.pi_engine_decode(self.handle, T, self.st))

    def advance(self, T: int):
        """tokens <- argmax, pos += 1 on the device (free-running greedy decode)."""
        check(lib.pi_engine_advance(self.handle, T, self.st))

    def device_view(self, what: str, T: int):
        """torch view of an engine I/O buffer: tokens / pos / argmax int32 [T], logits float32 [T, n_vocab]."""
        idx = {"tokens": 0, "pos": 1, "logits": 2, "argmax": 3}[what]
        n = T * self.spec.n_vocab if what == "logits" else T
        dt = torch.float32 if what == "logits" else torch.int32
        return _wrap_device(self.io[idx], n, dt).view(T, -1) if what == "logits" else _wrap_device(self.io[idx], n, dt)

    def profile_step(self, T: int):
        ms = (C.c_float * N_STAGES)()
        launches = C.c_int(0)
        check(lib.pi_engine_profile_step(self.handle, T, ms, C.byref(launches), self.st))
        return {STAGE_NAMES[i]: ms[i] for i in range(N_STAGES)}, launches.value

    def time_stage(self, T: int, stage: str, reps: int = 5):
        """(ms per launch, launches per replay) of one stage's kernels over all layers, back to back in a graph."""
        ms, launches = C.c_float(0), C.c_int(0)
        check(lib.pi_engine_time_stage(self.handle, T, STAGE_NAMES.index(stage), reps, C.byref(ms), C.byref(launches), self.st))
        return ms.value / max(1, launches.value), launches.value

    def active_total(self, reset: bool = True) -> int:
        v = C.c_uint64(0)
        check(lib.pi_engine_active_total(self.handle, 1 if reset else 0, C.byref(v), self.st))
        return v.value

    def launches(self) -> int:
        return lib.pi_engine_launches(self.handle)

    def status(self):
        check(lib.pi_engine_status(self.handle, self.st))

    def enable_trace(self):
        """Keep every layer's predictor logits of a step (tests compare active sets layer by layer)."""
        F = self.spec.n_ff // self.n_ranks
        self.trace = torch.zeros(self.spec.n_layer, self.max_batch, F, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        check(lib.pi_engine_set_trace(self.handle, self.trace.data_ptr()))

    def predictor_trace(self, T: int) -> np.ndarray:
        torch.cuda.synchronize()
        return self.trace[:, :T].cpu().numpy()

    def last_layer_predictor(self, T: int):
        pred, lst, cnt = _vp(), _vp(), _vp()
        check(lib.pi_engine_debug(self.handle, C.byref(pred), C.byref(lst), C.byref(cnt)))
        F = self.spec.n_ff // self.n_ranks
        torch.cuda.synchronize()
        n = int(_wrap_device(cnt.value, 1, torch.int32).item())
        return (_wrap_device(pred.value, T * F, torch.float32).view(T, F).cpu().numpy(),
                _wrap_device(lst.value, F, torch.int32)[:n].cpu().numpy())

    # ---- sharded runs: mailboxes in every rank's memory, addresses exchanged through the process group
    def _exchange_sizes(self):
        slot = self.max_batch * self.spec.d
        mbox_bytes = 2 * self.n_ranks * slot * 8          # pairs {value, number of the exchange}
        return slot, mbox_bytes, mbox_bytes + 256         # + the step counter

    def setup_exchange(self, group=None):
        import torch.distributed as dist
        assert self.n_ranks > 1
        slot, mbox_bytes, total = self._exchange_sizes()
        base = _vp()
        check(lib.pi_device_malloc(C.byref(base), total))
        handle = (C.c_char * 64)()
        check(lib.pi_ipc_export(base, handle))
        mine = torch.tensor(list(handle.raw), dtype=torch.uint8, device="cuda")
        allh = [torch.empty_like(mine) for _ in range(self.n_ranks)]
        dist.all_gather(allh, mine, group=group)
        x = Exchange()
        x.n_ranks, x.rank_id, x.slot_floats = self.n_ranks, self.rank, slot
        self._peer_ptrs = []
        for r in range(self.n_ranks):
            if r == self.rank:
                p = base.value
            else:
                hb = bytes(allh[r].cpu().tolist())
                pp = _vp()
                check(lib.pi_ipc_import(hb, C.byref(pp)))
                p = pp.value
                self._peer_ptrs.append(p)
            x.mailbox_peer[r] = p
        x.mailbox_local = base.value
        x.epoch = base.value + mbox_bytes
        self._xch_mem = base
        self.xch = x
        check(lib.pi_engine_set_exchange(self.handle, C.byref(x)))
        dist.barrier(group=group)

    def setup_exchange_loopback(self):
        """A sharded engine alone on one GPU (tests of the bounded waits): this rank's shares for the other ranks land in a
        spare buffer nobody reads, and nobody writes the other ranks' shares into this rank's mailbox, so every exchange
        wait runs out, unless `fill_peer_shares` is called."""
        assert self.n_ranks > 1
        slot, mbox_bytes, total = self._exchange_sizes()
        base, spare = _vp(), _vp()
        check(lib.pi_device_malloc(C.byref(base), total))
        check(lib.pi_device_malloc(C.byref(spare), total))
        x = Exchange()
        x.n_ranks, x.rank_id, x.slot_floats = self.n_ranks, self.rank, slot
        for r in range(self.n_ranks):
            x.mailbox_peer[r] = base.value if r == self.rank else spare.value
        x.mailbox_local = base.value
        x.epoch = base.value + mbox_bytes
        self._xch_mem, self._xch_spare, self._peer_ptrs = base, spare, []
        self._mbox_view = _wrap_device(base.value, 2 * self.n_ranks * slot * 2, torch.int32)
        self.xch = x
        check(lib.pi_engine_set_exchange(self.handle, C.byref(x)))

    def fill_peer_shares(self):
        """Loopback only: make every other rank's share read as delivered for all future exchanges (value 0.0 beside a
        number larger than any exchange's)."""
        mb = self._mbox_view.view(2, self.n_ranks, -1, 2)
        for r in range(self.n_ranks):
            if r != self.rank:
                mb[:, r, :, 0] = 0
                mb[:, r, :, 1] = 0x3fffffff
        torch.cuda.synchronize()

    def set_wait_cycles(self, cycles: int):
        check(lib.pi_engine_set_wait_cycles(self.handle, cycles))

    def close(self):
        if getattr(self, "handle", None) and self.handle.value:
            torch.cuda.synchronize()
            lib.pi_engine_destroy(self.handle)
            self.handle = _vp()
            for p in getattr(self, "_peer_ptrs", []):
                lib.pi_ipc_close(p)
            if self._xch_mem is not None:
                lib.pi_device_free(self._xch_mem)
                self._xch_mem = None
            if getattr(self, "_xch_spare", None) is not None:
                lib.pi_device_free(self._xch_spare)
                self._xch_spare = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _Cai:
    """Minimal __cuda_array_interface__ holder so torch can view memory the engine carved from its workspace."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}


def _wrap_device(ptr: int, n: int, dtype):
    return torch.as_tensor(_Cai(ptr, n, "<f4" if dtype == torch.float32 else "<i4"), device="cuda")
