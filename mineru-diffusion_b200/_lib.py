"""ctypes binding of libmdb200.so (the declarations of include/mdb200.h).

There is no fallback: if the library is missing or a call fails, this raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmdb200.so")

_p = C.c_void_p
_i = C.c_int
_i64 = C.c_int64
_u32 = C.c_uint32
_f = C.c_float

# name -> (restype, argtypes); mirrors include/mdb200.h one to one
SIGNATURES = {
    "mdb_strerror": (C.c_char_p, [_i]),
    "mdb_version": (_i, []),
    "mdb_set_option": (_i, [_i, _i]),
    "mdb_set_trace": (_i, [_p, _i64]),
    "mdb_get_option": (_i, [_i]),
    "mdb_last_device_status": (_i, [C.POINTER(C.c_uint), _i]),
    "mdb_kv_commit": (_i, [_p, _i64, _p, _i64, _p, _p, _p, _i, _i, _i64, _p]),
    "mdb_attn_paged_workspace_bytes": (_i64, [_i, _i, _i, _i]),
    "mdb_attn_block_paged": (_i, [_p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _f, _i, _p, _i64, _p]),
    "mdb_attn_block_paged_noalloc_limit": (_i64, []),
    "mdb_attn_block_paged_noalloc": (_i, [_p, _p, _p, _p, _p, _i, _p, _i, _i, _i, _i, _i, _f, _i, _p]),
    "mdb_attn_staircase_varlen": (_i, [_p, _i64, _p, _i64, _p, _i64, _p, _i64, _p, _i, _i, _i64, _i, _i, _i, _p]),
    "mdb_gemm_bf16": (_i, [_p, _i64, _p, _p, _i64, _i, _i, _i, _p]),
    "mdb_gemm_pick_ksplit": (_i, [_i, _i, _i]),
    "mdb_gemm_splitk_workspace_bytes": (_i64, [_i, _i, _i]),
    "mdb_gemm_splitk_partials": (_i, [_p, _i64, _p, _p, _i, _i, _i, _i, _p]),
    "mdb_gemm_gateup_swiglu": (_i, [_p, _i64, _p, _p, _i64, _i, _i, _i, _p]),
    "mdb_silu_mul": (_i, [_p, _i64, _p, _i64, _i, _i, _p]),
    "mdb_add_rmsnorm": (_i, [_p, _p, _i, _p, _p, _f, _p, _p, _i, _i, _p]),
    "mdb_qknorm_rope_commit": (_i, [_p, _i64, _p, _i, _p, _p, _i, _p, _p, _f, _p, _p, _p, _p, _p, _p, _i64, _i, _i,
                                    _i, _p]),
    "mdb_gemm_qkv_rope_commit": (_i, [_p, _i64, _p, _i, _i, _p, _p, _i, _p, _p, _f, _p, _p, _p, _p, _p, _p, _i64, _i, _i,
                                      _p]),
    "mdb_gather_rows": (_i, [_p, _i64, _p, _p, _i, _i, _p]),
    "mdb_lmhead_workspace_bytes": (_i64, [_i, _i]),
    "mdb_lmhead_sample": (_i, [_p, _i64, _p, _i, _i, _i, _p, _i, _i, _p, _u32, _u32, _p, _p, _i64, _p, _p, _p]),
    "mdb_logits_sample": (_i, [_p, _i64, _i, _i, _p, _i, _i, _p, _u32, _u32, _p, _p, _i64, _p, _p, _p]),
    "mdb_gumbel_noise": (_i, [_p, _i, _i, _u32, _u32, _p]),
    "mdb_unmask_decide": (_i, [_p, _p, _p, _i, _i, _i64, _f, _i, _p, _p, _p, _p, _p]),
    "mdb_tp_alloc": (_i, [_i64, C.POINTER(C.c_void_p)]),
    "mdb_tp_free": (_i, [_p]),
    "mdb_tp_export": (_i, [_p, _p]),
    "mdb_tp_import": (_i, [_p, C.POINTER(C.c_void_p)]),
    "mdb_tp_release": (_i, [_p]),
    "mdb_gemm_splitk_partials_tp": (_i, [_p, _i64, _p, _p, _p, _i, _i, _i, _i, _p, _u32, _p, _p]),
    "mdb_tp_grid_size": (_i, [_i, _i, _i, _i]),
    "mdb_add_rmsnorm_tp": (_i, [_p, _p, _i, _p, _p, _f, _p, _p, _i, _i, _p, _i, _u32, _p, _p]),
    "mdb_lmhead_tp_workspace_bytes": (_i64, [_i, _i]),
    "mdb_lmhead_tp_slots": (_i, [_i, _i]),
    "mdb_gemm_bf16_tp": (_i, [_p, _i64, _p, _p, _p, _i64, _i, _i, _i, _p, _u32, _p, C.POINTER(C.c_int), _p]),
    "mdb_add_rmsnorm_tp_rows": (_i, [_p, _p, _p, _p, _f, _p, _p, _i, _i, _p, _i, _u32, _p, _p]),
    "mdb_lmhead_sample_tp": (_i, [_p, _i64, _p, _i, _i, _i, _p, _i, _i, _p, _u32, _u32, _p, _p, _p, _i64, _i, _i, _p,
                                  _p, _i, _u32, _p, _p, _p, _p]),
}

_lib = None


class MdbError(RuntimeError):
    """A libmdb200 entry point returned a negative code."""


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python mineru-diffusion_b200/build.py` "
                "(there is no CPU or torch fallback for these ops)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().mdb_strerror(rc).decode()
        raise MdbError(f"{what}: {msg} (code {rc})")


def device_status(clear: bool = True) -> int:
    out = C.c_uint(0)
    check(lib().mdb_last_device_status(C.byref(out), 1 if clear else 0), "mdb_last_device_status")
    return int(out.value)
