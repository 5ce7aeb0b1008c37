"""ctypes binding of the attention-stage C ABI (``include/glinthawk_attn.h``).

There is no fallback of any kind: if the shared library is missing, importing this module raises, and every
compute entry point of the library launches CUDA kernels or returns an error status.
"""
from __future__ import annotations

import ctypes as C
import os
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("GLINTHAWK_ATTN_LIB", PKG / "libglinthawk_attn.so"))  # override for A/B runs
HEADERS = sorted((PKG.parent / "include").glob("*.h"))

GH_OK, GH_ERR_INVALID, GH_ERR_CUDA, GH_ERR_NO_SLOT, GH_ERR_CAPACITY = 0, 1, 2, 3, 4
GH_ERR_OOM, GH_ERR_UNSUPPORTED, GH_ERR_STATE, GH_ERR_NOT_FOUND = 5, 6, 7, 8
GH_F16, GH_F32, GH_BF16 = 0, 1, 2
GH_COPY_H2D, GH_COPY_D2H, GH_COPY_D2D, GH_COPY_H2H = 0, 1, 2, 3
GH_BACKING_STATIC, GH_BACKING_PAGED = 0, 1
GH_ROUTE_POSITION, GH_ROUTE_BALANCED = 0, 1


class Config(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("head_size", C.c_uint32), ("seq_len", C.c_uint32), ("n_layers_hosted", C.c_uint32),
                ("dtype", C.c_uint32), ("max_batch", C.c_uint32), ("max_contexts", C.c_uint32),
                ("backing", C.c_uint32), ("device", C.c_int32), ("decode_chunk", C.c_uint32),
                ("page_budget", C.c_uint64), ("force_generic", C.c_uint32), ("pipeline_steps", C.c_uint32)]


class NoallocShape(C.Structure):
    _fields_ = [("struct_size", C.c_uint32), ("n_heads", C.c_uint32), ("n_kv_heads", C.c_uint32),
                ("head_size", C.c_uint32), ("dtype", C.c_uint32)]


class Stats(C.Structure):
    _fields_ = [("kernel_launches", C.c_uint64), ("bytes_mapped", C.c_uint64), ("bytes_reserved", C.c_uint64),
                ("scratch_bytes", C.c_uint64), ("slots_free", C.c_uint32), ("slots_allocated", C.c_uint32),
                ("last_items", C.c_uint32), ("last_chunk", C.c_uint32), ("last_kernel", C.c_uint32),
                ("device_error", C.c_uint32), ("last_split_contexts", C.c_uint32), ("pad", C.c_uint32),
                ("batch_plans", C.c_uint64)]


_P, _U32, _U64, _I32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32
_PROTOS = {
    "gh_attn_create": (C.c_int, [C.POINTER(Config), C.POINTER(_P)]),
    "gh_attn_destroy": (C.c_int, [_P]),
    "gh_attn_last_error": (C.c_char_p, [_P]),
    "gh_status_string": (C.c_char_p, [C.c_int]),
    "gh_attn_get_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "gh_attn_synchronize": (C.c_int, [_P, _P]),
    "gh_attn_clear_device_error": (C.c_int, [_P]),
    "gh_attn_inject_device_error": (C.c_int, [_P, _U32]),
    "gh_attn_set_rope_tables": (C.c_int, [_P, _P, _P]),
    "gh_slot_acquire": (C.c_int, [_P, _U32, C.POINTER(_I32)]),
    "gh_slots_acquire_batch": (C.c_int, [_P, _U64, _P, _P]),
    "gh_slot_lookup": (C.c_int, [_P, _U32, C.POINTER(_I32)]),
    "gh_slot_release": (C.c_int, [_P, _U32]),
    "gh_slot_prepare": (C.c_int, [_P, _I32, _U32, _U32, C.c_int]),
    "gh_slot_layer_ptr": (C.c_int, [_P, _I32, _U32, C.POINTER(_P)]),
    "gh_slot_token_ptr": (C.c_int, [_P, _I32, _U32, _U32, C.POINTER(_P)]),
    "gh_slot_bytes": (C.c_size_t, [_P]),
    "gh_attn_batch_begin": (C.c_int, [_P, _U64, _P, _P, _P]),
    "gh_attn_append": (C.c_int, [_P, _U32, _P, _P, _P]),
    "gh_attn_decode": (C.c_int, [_P, _U32, _P, _P, _P]),
    "gh_attn_step": (C.c_int, [_P, _U32, _P, _P, _P, _P]),
    "gh_attn_prefill_chunk": (C.c_int, [_P, _U32, _U64, _P, _P, _U32, _P, _P, _P, _P]),
    "gh_attn_project_append": (C.c_int, [_P, _U32, _P, _P, _P, _P, _P, _P]),
    "gh_plan_projection": (C.c_int, [_U32, _U32, _U32, _U32, _P, _P, _U32, _P]),
    "gh_op_project_append": (C.c_int, [_P, _U64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "gh_attn_forward_attention_host": (C.c_int, [_P, _U32, _U32, _P, _P, _P, _P]),
    "gh_attn_forward_attention_state": (C.c_int, [_P, _U32, _P, C.c_size_t, _P]),
    "gh_op_copy_kv_cache": (C.c_int, [_P, _P, _P, _U64, _P]),
    "gh_op_apply_rope": (C.c_int, [_P, _U64, _P, _P, _P, _P, _P, _P]),
    "gh_op_copy_kv_cache_apply_rope": (C.c_int, [_P, _U64, _P, _P, _P, _P, _P, _P, _P]),
    "gh_op_attention_0_gemm": (C.c_int, [_P, _P, _P, _P, _U64, _P, _P]),
    "gh_op_attention_softmax": (C.c_int, [_P, _P, _P, _P, _U64, _P]),
    "gh_op_attention_2_gemm": (C.c_int, [_P, _P, _P, _P, _U64, _P, _P]),
    "gh_op_attention_fused": (C.c_int, [_P, _P, _P, _P, _U64, _P, _P]),
    "gh_op_convert_and_copy": (C.c_int, [_P, _P, _U32, _P, _U32, _U64, _U32]),
    "gh_fill_normal": (C.c_int, [_P, _P, _U64, _U32, _U64, _U64, _P]),
    "gh_decode_noalloc": (C.c_int, [C.POINTER(NoallocShape), _U64, _P, _P, _P, _P, _P]),
    "gh_decode_noalloc_error": (C.c_char_p, []),
    "gh_plan_batch": (C.c_int, [_U32, _U32, _U32, _U32, _U32, _U64, _P, _P, C.POINTER(_U32), C.POINTER(_U32)]),
    "gh_router_create": (C.c_int, [C.POINTER(_P), _U32, _U32, _U32, _U32]),
    "gh_router_destroy": (None, [_P]),
    "gh_router_is_context_available": (C.c_int, [_P]),
    "gh_router_assign_ranks": (C.c_int, [_P, _U32, _P, _P, _P]),
    "gh_router_lookup": (C.c_int, [_P, _U64, C.POINTER(_U32)]),
    "gh_router_note_tokens": (C.c_int, [_P, _U32, _P, _P]),
    "gh_router_release": (C.c_int, [_P, _U32, _P]),
    "gh_router_loads": (C.c_int, [_P, _P, _P]),
    "gh_router_cut": (C.c_int, [_U32, _U32, _P, _P, _P]),
}


def declared_symbols() -> list[str]:
    """Every function name the public headers declare."""
    names: set[str] = set()
    for header in HEADERS:
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(gh_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m glinthawk_b200.build` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in _PROTOS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = load()
