"""ctypes binding of libadaptq_b200.so (the C ABI declared in include/*.h).

The library is the product; this module only loads it.  There is no fallback:
if the shared object is missing or cannot be loaded, importing fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ADAPTQ_B200_LIB") or os.path.join(_HERE, "libadaptq_b200.so")

f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)
i8p = C.POINTER(C.c_int8)
intp = C.POINTER(C.c_int)


class MhaInfo(C.Structure):
    _fields_ = [("n_heads", C.c_int), ("dim", C.c_int), ("padded", C.c_int), ("k_bits", C.c_int),
                ("v_bits", C.c_int), ("capacity", C.c_int), ("hybrid_thresh", C.c_int),
                ("k_row_bytes", C.c_int), ("v_row_bytes", C.c_int), ("device", C.c_int),
                ("v_mass", C.c_float), ("device_bytes", C.c_size_t)]


# name -> (restype, argtypes); every symbol declared in include/*.h
SYMBOLS = {
    "adaptq_last_error": (C.c_char_p, []),
    "adaptq_create": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_float, C.c_int]),
    "adaptq_destroy": (None, [C.c_void_p]),
    "adaptq_append": (None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "adaptq_compute": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "adaptq_compute_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "adaptq_reset": (None, [C.c_void_p]),
    "adaptq_kv_bytes": (C.c_size_t, [C.c_void_p]),
    "adaptq_mha_create": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_float, C.c_int]),
    "adaptq_mha_destroy": (None, [C.c_void_p]),
    "adaptq_mha_append": (None, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int]),
    "adaptq_mha_compute": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "adaptq_mha_compute_batch": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "adaptq_mha_reset": (None, [C.c_void_p]),
    "adaptq_mha_total_kv_bytes": (C.c_size_t, [C.c_void_p]),
    "adaptq_features": (C.c_uint, []),
    "adaptq_version": (C.c_char_p, []),
    "adaptq_mha_create_seeded": (C.c_void_p, [C.c_int, C.POINTER(C.c_uint64), C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]),
    "adaptq_mha_append_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "adaptq_mha_compute_all": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "adaptq_mha_compute_all_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "adaptq_mha_compute_partial_to_peers": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p),
                                                       C.POINTER(C.c_void_p), C.c_int, C.c_int]),
    "adaptq_mha_merge_from_peers": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_uint, C.c_int, C.c_void_p]),
    "adaptq_mha_decode_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "adaptq_mha_partial_floats": (C.c_int, [C.c_void_p]),
    "adaptq_mha_compute_partial": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "adaptq_mha_merge_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "adaptq_mha_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "adaptq_mha_synchronize": (C.c_int, [C.c_void_p]),
    "adaptq_mha_info": (C.c_int, [C.c_void_p, C.POINTER(MhaInfo)]),
    "adaptq_mha_export_head": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_void_p, intp, intp, intp]),
    "adaptq_stack_create": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.c_uint64,
                                         C.c_float, C.c_int]),
    "adaptq_stack_destroy": (None, [C.c_void_p]),
    "adaptq_stack_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "adaptq_stack_compute": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "adaptq_stack_decode_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "adaptq_stack_reset": (C.c_int, [C.c_void_p]),
    "adaptq_stack_kv_bytes": (C.c_size_t, [C.c_void_p]),
    "adaptq_stack_parts": (C.c_int, [C.c_void_p]),
    "adaptq_stack_layer_handle": (C.c_void_p, [C.c_void_p, C.c_int, intp]),
    "adaptq_stack_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "adaptq_stack_synchronize": (C.c_int, [C.c_void_p]),
    # include/adaptq_runtime.h
    "adaptq_runtime_create": (C.c_void_p, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]),
    "adaptq_runtime_destroy": (None, [C.c_void_p]),
    "adaptq_runtime_append": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "adaptq_runtime_compute": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "adaptq_runtime_append_token": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "adaptq_runtime_compute_token": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "adaptq_runtime_reset": (C.c_int, [C.c_void_p]),
    "adaptq_runtime_token_pos": (C.c_int, [C.c_void_p]),
    "adaptq_runtime_handle": (C.c_void_p, [C.c_void_p]),
    "adaptq_runtime_snapshot_save": (C.c_int, [C.c_void_p, C.c_char_p]),
    "adaptq_runtime_snapshot_load": (C.c_void_p, [C.c_char_p, C.c_int, C.c_float]),
    "adaptq_mha_import_head": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int, C.c_int, C.c_int]),
    "adaptq_kernel_fwht_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "adaptq_kernel_fwht_inverse": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "adaptq_kernel_kdot_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "adaptq_kernel_vaccum_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "adaptq_kernel_backend_name": (C.c_char_p, []),
    "adaptq_inject_failure": (C.c_int, [C.c_int, C.c_int]),
    "adaptq_kernel_launches": (C.c_ulonglong, []),
    "adaptq_set_kernel_policy": (C.c_int, [C.c_int]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library and type its entry points.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found. Build it with `python -m adaptq_b200.build` "
            "(needs nvcc; the library targets sm_100a and has no CPU fallback).")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError here = the library is missing a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().adaptq_last_error().decode("utf-8", "replace")
