"""ctypes binding of ``libmorphkv.so`` (declared in ``include/morphkv.h``).

There is no fallback: importing this module raises if the CUDA library has not
been built (``python morphserve_b200/build.py``), and every wrapper raises on a
non-zero status.  Argument errors keep the reference's exception types at the
Python layer (the callers translate), everything else is a RuntimeError.
"""
from __future__ import annotations

import ctypes as C
import os

MKV_MAX_SEGMENTS = 65
# MORPHKV_LIB names another build of the same library (a debug or instrumented build); default: the in-tree one
_LIB_PATH = os.environ.get("MORPHKV_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libmorphkv.so")

if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} is missing: build the CUDA library first (python morphserve_b200/build.py). "
        "morphserve_b200 has no CPU or Triton fallback.")

lib = C.CDLL(_LIB_PATH)


class MkvPool(C.Structure):
    _fields_ = [
        ("num_segments", C.c_int32),
        ("elem_bytes", C.c_int32),
        ("num_layers", C.c_int32),
        ("num_kv_heads", C.c_int32),
        ("block_size", C.c_int32),
        ("head_dim", C.c_int32),
        ("num_blocks_org", C.c_int64),
        ("chunk_blocks", C.c_int64),
        ("k_base", C.c_void_p * MKV_MAX_SEGMENTS),
        ("v_base", C.c_void_p * MKV_MAX_SEGMENTS),
    ]


_vp, _i, _i64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float
_pool = C.POINTER(MkvPool)

# name -> (restype, argtypes); must list every function of include/morphkv.h
SIGNATURES = {
    "mkv_version": (_i, []),
    "mkv_status_string": (C.c_char_p, [_i]),
    "mkv_last_cuda_error": (C.c_char_p, []),
    "mkv_sm_count": (_i, [_i, C.POINTER(_i)]),
    "mkv_attn_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i]),
    "mkv_attn_plan": (_i, [_i, _vp, _vp, _sz, _vp, _vp, _i, _i, _i, _i, _i, _i]),
    "mkv_attn_configure": (_i, [_i, _i, C.c_double, C.c_double, _i]),
    "mkv_attn_set_static_deal": (_i, [_i, _i, _i]),
    "mkv_attn_workspace_layout": (_i, [_i, _i, _i, _i, _i, _i, C.POINTER(_i64)]),
    "mkv_paged_attention_decode_push": (_i, [_i, _vp, _vp, C.POINTER(_vp), _i, _i64, _i64, C.POINTER(_vp), _i, C.c_int32,
                                             _vp, _vp, _pool, _vp, _i64, _vp, _vp, _i, _i, _i, _f, _i, _vp, _sz]),
    "mkv_wait_ready": (_i, [_i, _vp, _vp, _i, C.c_int32, _i64, _vp]),
    "mkv_paged_attention_decode_append": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp, _i, _i, _i, _f,
                                               _i, _vp, _sz]),
    "mkv_paged_attention_decode": (_i, [_i, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp, _i, _i, _i, _f, _i, _vp, _sz]),
    "mkv_attn_read_error_flags": (_i, [_i, _vp, _vp, C.POINTER(_i)]),
    "mkv_paged_attention_decode_noalloc": (_i, [_i, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp, _i, _i, _i, _f, _i]),
    "mkv_noalloc_scratch_bytes": (_sz, []),
    "mkv_rotary_embedding": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i]),
    "mkv_rope_set_rounding": (_i, [_i]),
    "mkv_paged_attention_decode_rope_append": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp,
                                                   _i, _i, _i, _f, _i, _vp, _sz]),
    "mkv_store_kv_decode": (_i, [_i, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp, _i, _i]),
    "mkv_store_kv_prefill": (_i, [_i, _vp, _vp, _vp, _pool, _vp, _i64, _vp, _vp, _vp, _i, _i, _i]),
    "mkv_block_need": (_i, [_i, _vp, _vp, _i, _vp, _vp, _i, _i, _vp, _vp]),
    "mkv_slab_upload": (_i, [_i, _vp, _sz, _vp, _sz]),
    "mkv_block_allocate": (_i, [_i, _vp, _vp, _i, _vp, _i64, _vp, _vp, _i, _i, _vp, _i64, _vp, _vp, _i64, _vp]),
    "mkv_bitmap_select": (_i, [_i, _vp, _vp, _i64, _i64, _i, _i64, _i, _vp, _vp, _vp]),
    "mkv_bitmap_scatter": (_i, [_i, _vp, _vp, _i64, _vp, _i64, _i]),
    "mkv_block_table_set": (_i, [_i, _vp, _vp, _i, _vp, _i64, _vp, _vp, _vp, _i]),
    "mkv_block_table_unset": (_i, [_i, _vp, _vp, _i, _vp, _i64, _vp, _i, _vp, _i64, _vp, _i64, _vp, _i]),
    "mkv_block_table_count": (_i, [_i, _vp, _vp, _i, _vp, _i, _vp]),
    "mkv_chunk_layout": (_i, [C.c_uint64, C.c_uint64, C.c_uint64, _i, _i, _i, _i, _i,
                              C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(_i64)]),
    "mkv_copy_blocks": (_i, [_i, _vp, _pool, _vp, _vp, _i64]),
    "mkv_remap_block_table": (_i, [_i, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64]),
    "mkv_compact_plan": (_i, [_i, _vp, _vp, _i64, _i64, _vp, _vp, _i64, _vp]),
    "mkv_copy_blocks_counted": (_i, [_i, _vp, _pool, _vp, _vp, _i64, _vp]),
    "mkv_remap_block_table_counted": (_i, [_i, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "mkv_swap_blocks": (_i, [_i, _vp, _pool, _vp, _vp, _i64, C.POINTER(_i64), C.POINTER(_i64), _i64, _i,
                             C.POINTER(_i64)]),
    "mkv_swap_blocks_pinned": (_i, [_i, _vp, _pool, _vp, _vp, _i64, _vp, _vp, _i64, _i]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError here = library and header disagree
    _fn.restype = _res
    _fn.argtypes = _args


class MorphKVError(RuntimeError):
    def __init__(self, status: int, where: str):
        msg = lib.mkv_status_string(status).decode()
        if status == -6:
            msg += ": " + lib.mkv_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (status {status})")
        self.status = status


CALLS: dict = {}   # entry point -> number of successful calls (each kernel entry point = one launch)


def check(status: int, where: str) -> None:
    if status != 0:
        raise MorphKVError(status, where)
    CALLS[where] = CALLS.get(where, 0) + 1


def sm_count(device: int) -> int:
    n = C.c_int(0)
    check(lib.mkv_sm_count(device, C.byref(n)), "mkv_sm_count")
    return n.value
