"""ctypes wrapper of the native (C++) reader for the reference's model and placement files: `pi_model_file_*` in
include/powerinfer_b200.h.  Host only.  `gguf_loader.py` is the numpy reader the engine driver uses; this one is what a
C or C++ host links, bound here so that the tests can hold the two against each other."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import check, lib
from .engine import EngineConfig

_vp = C.c_void_p
MODEL_FILE_EXPORTS = ["pi_model_file_open", "pi_model_file_close", "pi_model_file_is_powerinfer", "pi_model_file_get_u64",
                      "pi_model_file_get_f32", "pi_model_file_get_str", "pi_model_file_n_tensors", "pi_model_file_tensor_at",
                      "pi_model_file_tensor", "pi_model_file_engine_config"]

for _name, _res, _args in [
    ("pi_model_file_open", C.c_int, [C.c_char_p, C.POINTER(_vp)]),
    ("pi_model_file_close", None, [_vp]),
    ("pi_model_file_is_powerinfer", C.c_int, [_vp]),
    ("pi_model_file_get_u64", C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    ("pi_model_file_get_f32", C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_float)]),
    ("pi_model_file_get_str", C.c_int, [_vp, C.c_char_p, C.POINTER(_vp), C.POINTER(C.c_size_t)]),
    ("pi_model_file_n_tensors", C.c_int64, [_vp]),
    ("pi_model_file_tensor_at", C.c_int, [_vp, C.c_int64, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int64 * 4),
                                          C.POINTER(_vp), C.POINTER(C.c_size_t)]),
    ("pi_model_file_tensor", C.c_int, [_vp, C.c_char_p, C.POINTER(C.c_int), C.POINTER(C.c_int64 * 4), C.POINTER(_vp),
                                       C.POINTER(C.c_size_t)]),
    ("pi_model_file_engine_config", C.c_int, [_vp, C.POINTER(EngineConfig)]),
]:
    _fn = getattr(lib, _name)
    _fn.restype, _fn.argtypes = _res, _args


class ModelFile:
    def __init__(self, path: str):
        self.h = _vp()
        check(lib.pi_model_file_open(path.encode(), C.byref(self.h)))

    def close(self):
        if self.h:
            lib.pi_model_file_close(self.h)
            self.h = _vp()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def is_powerinfer(self) -> bool:
        return bool(lib.pi_model_file_is_powerinfer(self.h))

    def u64(self, key: str) -> int:
        v = C.c_uint64()
        check(lib.pi_model_file_get_u64(self.h, key.encode(), C.byref(v)))
        return v.value

    def f32(self, key: str) -> float:
        v = C.c_float()
        check(lib.pi_model_file_get_f32(self.h, key.encode(), C.byref(v)))
        return v.value

    def string(self, key: str) -> str:
        p, n = _vp(), C.c_size_t()
        check(lib.pi_model_file_get_str(self.h, key.encode(), C.byref(p), C.byref(n)))
        return C.string_at(p, n.value).decode("utf-8", errors="replace")

    def _unpack(self, ty, ne, data, nbytes):
        raw = np.frombuffer(C.string_at(data, nbytes.value), np.uint8) if nbytes.value else None
        return ty.value, tuple(ne), raw

    def tensors(self) -> dict:
        """name -> (ggml type, ne[4], bytes as a uint8 array, or None for a type the reader has no size for)"""
        out = {}
        for i in range(lib.pi_model_file_n_tensors(self.h)):
            name, ty, ne, data, nbytes = C.c_char_p(), C.c_int(), (C.c_int64 * 4)(), _vp(), C.c_size_t()
            check(lib.pi_model_file_tensor_at(self.h, i, C.byref(name), C.byref(ty), C.byref(ne), C.byref(data), C.byref(nbytes)))
            out[name.value.decode("utf-8", errors="replace")] = self._unpack(ty, ne, data, nbytes)
        return out

    def tensor(self, name: str):
        ty, ne, data, nbytes = C.c_int(), (C.c_int64 * 4)(), _vp(), C.c_size_t()
        check(lib.pi_model_file_tensor(self.h, name.encode(), C.byref(ty), C.byref(ne), C.byref(data), C.byref(nbytes)))
        return self._unpack(ty, ne, data, nbytes)

    def engine_config(self) -> EngineConfig:
        cfg = EngineConfig()
        check(lib.pi_model_file_engine_config(self.h, C.byref(cfg)))
        return cfg
