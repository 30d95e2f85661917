"""ctypes binding of libxattn_b200.so (the C ABI declared in include/xattn_b200.h).

There is no fallback: if the library is missing or fails to load, importing an op raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libxattn_b200.so")

BF16, F16 = 0, 1
SEMANTICS_TORCH, SEMANTICS_TRITON, SEMANTICS_TORCH_BAND = 0, 1, 2

_i, _i64, _f, _d, _p, _sz = C.c_int, C.c_int64, C.c_float, C.c_double, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "xattn_b200_version": (_i, []),
    "xattn_b200_error_string": (C.c_char_p, [_i]),
    "xattn_b200_launch_count": (C.c_ulonglong, []),
    "xattn_b200_block_sparse_attn_split_share": (_i, [_i]),
    "xattn_b200_default_chunk_size": (_i, [_i]),
    "xattn_b200_estimate_geometry": (_i, [_i, _i, _i, _i, _i, C.POINTER(_i)]),
    "xattn_b200_estimate_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i]),
    "xattn_b200_estimate_workspace_bytes_ex": (_sz, [_i, _i, _i, _i, _i, _i, _i, _i, _i]),
    "xattn_b200_estimate": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                                 _i, _i, _i, _f, _i, _i, _p, _p, _sz, _p, _p]),
    "xattn_b200_estimate_static": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                                        _i, _i, _i, _f, _i, _i, _p, _p, _p]),
    "xattn_b200_split_f32": (_i, [_p, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i, _p, _p]),
    "xattn_b200_rope_qk": (_i, [_p, _p, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _p, _p, _i64, _i64, _p]),
    "xattn_b200_select": (_i, [_p, _i, _i, _i, _i, _i, _i, _i, _i, _d, _p, _i, _i, _p, _p, _p,
                               _i, _i, _i, _i, _p, _p]),
    "xattn_b200_select_band": (_i, [_p, _i, _i, _i, _i, _i, _i, _i, _i, _d, _p, _i, _i, _p, _p, _p,
                                    _i, _i, _i, _i, _p, _p]),
    "xattn_b200_mask_to_lists": (_i, [_p, _i, _i, _i, _i, _i, _i, _i, _p, _p, _p]),
    "xattn_b200_block_sparse_attn": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i,
                                          _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                          _p, _p, _i, _f, _p, _i64, _i64, _i64, _p, _p]),
    "xattn_b200_block_sparse_attn_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "xattn_b200_block_sparse_attn_ws": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i,
                                             _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                             _p, _p, _i, _f, _p, _i64, _i64, _i64, _p, _sz, _p, _p]),
}

_lib = None


class XattnB200Error(RuntimeError):
    pass


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise XattnB200Error(
            f"{LIB_PATH} is missing: build it with `python -m xattn_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().xattn_b200_error_string(code).decode()
        raise XattnB200Error(f"{what}: {msg} (status {code})")
