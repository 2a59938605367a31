"""ctypes binding of libmustafar_b200.so (the C ABI declared in include/mustafar_b200.h).

There is no fallback: if the shared library is missing the import of any op
raises, telling the user to build it (``python -m mustafar_b200.build``).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmustafar_b200.so")

OK = 0
DEV_CAPACITY, DEV_TIMEOUT, DEV_BADMETA = 1, 2, 4

_vp, _i64, _i32, _sz, _f32 = C.c_void_p, C.c_int64, C.c_int, C.c_size_t, C.c_float

# name -> (restype, argtypes); the order mirrors include/mustafar_b200.h
SIGNATURES = {
    "mfar_version": (_i32, []),
    "mfar_status_string": (C.c_char_p, [_i32]),
    "mfar_compress_scratch_bytes": (_sz, [_i32, _i32]),
    "mfar_compress_fp16": (_i32, [_vp, _i64, _i64, _i32, _i64, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _i64,
                                  _vp, _vp, _i64, _i64, _vp, _sz, _vp, _vp, _vp]),
    "mfar_compress_fp16_noalloc": (_i32, [_vp, _i64, _i64, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _i64, _i64,
                                          _vp, _vp, _i64, _i64, _vp, _vp, _vp]),
    "mfar_compact_heads_fp16": (_i32, [_vp, _i64, _vp, _i64, _i64, _i32, _vp, _i64, _vp]),
    "mfar_prune_fp16": (_i32, [_vp, _vp, _i64, _i64, _i32, _vp]),
    "mfar_compress_quant": (_i32, [_vp, _i64, _i64, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _vp, _vp, _vp, _vp, _vp,
                                   _i64, _i64, _vp, _i64, _i64, _vp, _vp, _sz, _vp, _vp]),
    "mfar_decode_plan": (_i32, [_i32, _i32, _i32, _i32, C.POINTER(_i32), C.POINTER(_sz), _i32]),
    "mfar_decode_attention_fp16": (_i32, [_vp, _i64, _i32, _i32,
                                          _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64,
                                          _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64,
                                          _i32, _vp, _vp, _i64, _i64, _i32, _vp, _f32, _vp, _i64, _vp, _sz,
                                          _i32, _i32, _vp, _vp]),
    "mfar_decode_attention_fp16_dyn": (_i32, [_vp, _i64, _i32, _i32,
                                              _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64,
                                              _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64,
                                              _i32, _vp, _vp, _vp, _i64, _i64, _i32, _vp, _f32, _vp, _i64, _vp, _sz,
                                              _i32, _i32, _vp, _vp]),
    "mfar_key_scores_fp16": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i32,
                                    _vp, _i64, _i32, _vp, _vp]),
    "mfar_value_output_fp16": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _i32,
                                      _vp, _i64, _vp, _sz, _i32, _i32, _vp, _vp]),
    "mfar_key_scores_quant": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i32, _i32, _i32,
                                     _vp, _i64, _vp, _vp]),
    "mfar_value_output_quant": (_i32, [_vp, _i64, _i32, _i32, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i32, _i32, _i32,
                                       _vp, _i64, _vp, _sz, _i32, _vp, _vp]),
    "mfar_decode_attention_quant": (_i32, [_vp, _i64, _i32, _i32,
                                           _vp, _vp, _vp, _vp, _vp, _i64,
                                           _vp, _vp, _vp, _vp, _vp, _i64,
                                           _i64, _i64, _i32, _vp, _i32, _i32,
                                           _vp, _vp, _i64, _i64, _i32, _vp,
                                           _f32, _vp, _i64, _vp, _sz, _i32, _vp, _vp]),
    "mfar_add_rmsnorm_f16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp]),
    "mfar_rope_append_f16": (_i32, [_vp, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i64, _i64, _i32, _i32,
                                    _i32, _vp, _vp]),
    "mfar_peer_argmax_f16": (_i32, [_vp, _i64, _i64, _i32, _i32, _vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _vp, _i64, _vp, _vp]),
    "mfar_peer_alloc": (_i32, [_i64, C.POINTER(C.c_void_p), C.c_void_p]),
    "mfar_peer_open": (_i32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "mfar_peer_close": (_i32, [C.c_void_p]),
    "mfar_peer_free": (_i32, [C.c_void_p]),
    "mfar_peer_reduce_add_rmsnorm_f16": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _vp, _vp, _i64, _i32, _f32,
                                                _i64, _vp, _vp]),
    "mfar_silu_mul_f16": (_i32, [_vp, _vp, _i64, _i32, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mustafar_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


class MustafarError(RuntimeError):
    pass


def check(status: int, what: str = "") -> None:
    if status != OK:
        msg = lib().mfar_status_string(status).decode()
        raise MustafarError(f"{what}: {msg} (status {status})" if what else f"{msg} (status {status})")


def check_dev_status(word: int, what: str = "") -> None:
    if word:
        names = [n for b, n in ((DEV_CAPACITY, "packed-value capacity exceeded"),
                                (DEV_TIMEOUT, "bounded wait timed out"),
                                (DEV_BADMETA, "inconsistent cache offsets / stage too small")) if word & b]
        raise MustafarError(f"{what}: device reported {', '.join(names)} (dev_status {word})")
