"""ctypes binding of libturbovec_b200.so.  There is no fallback: if the library is missing or a CUDA
device cannot be opened, the caller gets an exception."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libturbovec_b200.so")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_u64p = C.POINTER(C.c_uint64)
_i64p = C.POINTER(C.c_int64)
_szp = C.POINTER(C.c_size_t)
_intp = C.POINTER(C.c_int)
_H = C.c_void_p

# name -> (restype, argtypes); every symbol declared in include/turbovec_b200.h
SIGNATURES = {
    "tv_version": (C.c_char_p, []),
    "tv_exchange_layout_conflicts": (C.c_int, [C.c_size_t] + [C.POINTER(C.c_int)] * 4),
    "tv_search_device_keys": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_uint64, C.c_void_p, C.POINTER(C.c_size_t)]),
    "tv_merge_keys_device": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tv_merge_keys_device_chunked": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "tv_idtable_create": (C.c_int, [C.POINTER(_H)]),
    "tv_idtable_destroy": (None, [_H]),
    "tv_idtable_len": (C.c_size_t, [_H]),
    "tv_idtable_last_error": (C.c_char_p, [_H, _u64p]),
    "tv_idtable_add": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_idtable_truncate": (C.c_int, [_H, C.c_size_t]),
    "tv_idtable_remove": (C.c_int, [_H, C.c_uint64, _intp, _u64p, _u64p]),
    "tv_idtable_contains": (C.c_int, [_H, C.c_uint64, _intp]),
    "tv_idtable_resolve": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tv_idtable_ids_of": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tv_idtable_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_multi_create": (C.c_int, [C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_size_t, C.POINTER(_H)]),
    "tv_multi_destroy": (None, [_H]),
    "tv_multi_last_error": (C.c_char_p, [_H]),
    "tv_multi_error_id": (C.c_uint64, [_H]),
    "tv_multi_len": (C.c_size_t, [_H]),
    "tv_multi_shards": (C.c_int, [_H]),
    "tv_multi_shard": (_H, [_H, C.c_int]),
    "tv_multi_add": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t]),
    "tv_multi_add_with_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "tv_multi_swap_remove": (C.c_int, [_H, C.c_size_t, _szp]),
    "tv_multi_remove": (C.c_int, [_H, C.c_uint64, C.POINTER(C.c_int)]),
    "tv_multi_contains": (C.c_int, [_H, C.c_uint64, C.POINTER(C.c_int)]),
    "tv_multi_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_multi_search": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
    "tv_multi_search_allowlist": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
    "tv_quantise_grid_lookup": (C.c_int, [C.POINTER(C.c_float), C.c_int, C.POINTER(C.c_float), C.c_size_t, C.POINTER(C.c_uint8)]),
    "tv_index_create": (C.c_int, [C.c_size_t, C.c_int, C.c_int, C.c_int, C.POINTER(_H)]),
    "tv_index_destroy": (None, [_H]),
    "tv_last_error": (C.c_char_p, [_H]),
    "tv_error_detail": (None, [_H, _szp, _szp, _f32p, _u64p]),
    "tv_len": (C.c_size_t, [_H]),
    "tv_dim": (C.c_size_t, [_H]),
    "tv_bit_width": (C.c_int, [_H]),
    "tv_kind": (C.c_int, [_H]),
    "tv_set_option": (C.c_int, [_H, C.c_int, C.c_int64]),
    "tv_get_option": (C.c_int64, [_H, C.c_int]),
    "tv_add": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t]),
    "tv_add_with_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "tv_add_device": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t]),
    "tv_add_with_ids_device": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "tv_swap_remove": (C.c_int, [_H, C.c_size_t, _szp]),
    "tv_remove": (C.c_int, [_H, C.c_uint64, _intp]),
    "tv_get_row": (C.c_int, [_H, C.c_size_t, C.c_void_p, C.c_size_t, _f32p]),
    "tv_set_row": (C.c_int, [_H, C.c_size_t, C.c_void_p, C.c_size_t, C.c_float]),
    "tv_contains": (C.c_int, [_H, C.c_uint64, _intp]),
    "tv_ids": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_search": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                            C.c_void_p, C.c_void_p, _szp]),
    "tv_search_mask_words": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                       C.c_void_p, C.c_void_p, _szp]),
    "tv_search_allowlist": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                      C.c_void_p, C.c_void_p, _szp]),
    "tv_search_device": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, _szp]),
    "tv_search_device_noalloc": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
    "tv_mask_prepare_device": (C.c_int, [_H, C.c_void_p]),
    "tv_mask_prepare_words": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_mask_prepare_allowlist": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_search_prepared": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, _szp]),
    "tv_search_device_prepared": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, _szp]),
    "tv_prepare": (C.c_int, [_H]),
    "tv_blocked_bytes": (C.c_size_t, [_H]),
    "tv_export_blocked": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t]),
    "tv_export_packed": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_import_packed": (C.c_int, [_H, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "tv_crc32c": (C.c_uint32, [C.c_void_p, C.c_size_t]),
    "tv_image_bytes": (C.c_size_t, [_H]),
    "tv_to_bytes": (C.c_int, [_H, C.c_void_p, C.c_size_t]),
    "tv_from_bytes": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.POINTER(_H)]),
    "tv_write": (C.c_int, [_H, C.c_char_p]),
    "tv_load": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.POINTER(_H)]),
    "tv_sync": (C.c_int, [_H, C.c_char_p]),
    "tv_v7_plan_sync": (C.c_int, [C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p,
                                 C.POINTER(C.c_size_t), C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "tv_sync_state": (C.c_int, [_H, C.POINTER(C.c_int), C.POINTER(C.c_uint64), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "tv_codebook": (C.c_int, [_H, C.c_void_p, C.c_void_p]),
    "tv_rotate": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "tv_calibrate": (C.c_int, [_H, C.c_void_p, C.c_size_t, C.c_size_t]),
    "tv_calibration": (C.c_int, [_H, C.c_void_p, C.c_void_p, C.c_size_t, _intp]),
    "tv_set_calibration": (C.c_int, [_H, C.c_size_t, C.c_void_p, C.c_void_p]),
    "tv_measure_int8_peak": (C.c_int, [C.c_int, C.POINTER(C.c_double)]),
    "tv_measure_int8_peak_for": (C.c_int, [C.c_int, C.c_double, C.POINTER(C.c_double)]),
    "tv_launch_count": (C.c_uint64, [_H]),
    "tv_last_kernel_ms": (C.c_float, [_H]),
    "tv_last_main_kernel_ms": (C.c_float, [_H, _intp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m turbovec_b200.build` (needs nvcc). "
            "turbovec_b200 has no CPU implementation to fall back to.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


# status codes of include/turbovec_b200.h
OK = 0
ERR_ID_KEYERROR = {21}
ERR_INDEXERROR = {31}
SCORE_AUTO, SCORE_PERMUTE_DOT, SCORE_LUT_MULADD, SCORE_LUT_FLUSH = 0, 1, 2, 3
OPT_SCORE_MODE, OPT_MMA_MIN_BATCH, OPT_FORCE_CAREFUL, OPT_TC_TILES, OPT_INGEST_PIPELINE, OPT_PD_SPLIT = 1, 2, 3, 4, 5, 6
OPT_SMALL_SCAN, OPT_FAIL_NEXT, OPT_TC_WIDE, OPT_TC_EXPANDED, OPT_EXPANDED_BYTES, OPT_DENSE_PAIR = 7, 8, 10, 11, 12, 13
