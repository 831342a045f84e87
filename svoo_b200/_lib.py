"""ctypes binding of libsvoo_b200.so (the C ABI declared in include/svoo_b200.h).

There is no fallback: if the library is missing or a symbol is absent, importing
this module raises, and every op of the package raises with it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p, POINTER

from . import build as _build

_I64P = POINTER(c_int64)
_I32P = POINTER(c_int32)

# name -> (restype, argtypes); must list every function include/svoo_b200.h declares
SIGNATURES = {
    "svoo_b200_version": (c_int, []),
    "svoo_b200_error_string": (c_char_p, [c_int]),
    "svoo_b200_launch_count": (c_int64, []),
    "svoo_b200_workspace_bytes": (c_int, [c_int64, c_int64, c_int64, c_int64, _I64P]),
    "svoo_b200_cocluster": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                    c_int64, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_cocluster_assign": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                           c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_euclid_assign": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int64,
                                        c_void_p]),
    "svoo_b200_append_text_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                             c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p]),
    "svoo_b200_sort_labels": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_void_p]),
    "svoo_b200_sort_labels_static": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "svoo_b200_centroid_update": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                          c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_permute": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "svoo_b200_inverse_permute": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                          c_void_p]),
    "svoo_b200_block_map": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_float,
                                    _I32P, _I32P, c_void_p, c_void_p]),
    "svoo_b200_sparse_attn": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                      c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                      c_void_p]),
    "svoo_b200_sparse_attn_simt": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                           c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_int64,
                                           c_void_p]),
    "svoo_b200_status_offset": (c_int, [c_int64, c_int64, c_int64, c_int64, _I64P]),
    "svoo_b200_qk_prep_heads": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                        c_void_p, c_int64, c_int64, c_void_p]),
    "svoo_b200_ear_workspace_bytes": (c_int, [c_int64, c_int64, c_int64, c_int64, _I64P, _I64P]),
    "svoo_b200_ear_value_centroids": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p,
                                              c_void_p, c_int64, c_void_p]),
    "svoo_b200_ear_block_scores": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                           c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_ear_select_blocks": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float,
                                            _I32P, _I32P, c_void_p, c_void_p]),
    "svoo_b200_sparse_attn_ear_push": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                               c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p, c_int32, c_int64,
                                               c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_sparse_attn_ear": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                          c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int64, c_void_p]),
    "svoo_b200_offsets_from_sizes": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "svoo_b200_sparse_attn_push": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                           c_int64, c_int64, c_int64, c_float, c_void_p, c_void_p, c_int32, c_int64,
                                           c_int64, c_void_p, c_void_p, c_int64, c_void_p]),
    "svoo_b200_layer_scratch_bytes": (c_int, [c_int64, c_int64, c_int64, c_int64, c_int64, _I64P]),
    "svoo_b200_layer": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64,
                                c_int32, c_float, c_void_p, c_void_p, c_float, c_int64, c_int64, c_void_p, c_void_p, c_int64,
                                c_void_p, c_int64, c_void_p]),
    "svoo_b200_qk_prep": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_void_p,
                                  c_void_p]),
    "svoo_b200_qk_prep_push": (c_int, [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                       c_int32, c_int64, c_int64, c_int64, c_void_p]),
    "svoo_b200_peer_barrier": (c_int, [c_void_p, c_int32, c_int32, c_int32, ctypes.c_uint32, c_void_p, c_void_p]),
    "svoo_b200_push_heads": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int64, c_int64, c_int64,
                                     c_void_p]),
    "svoo_b200_push_seq": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int64, c_int64, c_void_p]),
}


VERSION = 104          # SVOO_B200_VERSION of include/svoo_b200.h this binding was written for


class SvooB200Error(RuntimeError):
    """A non-zero status from the C ABI."""


def _load() -> ctypes.CDLL:
    path = _build.LIB_PATH
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m svoo_b200.build` (needs nvcc); "
            "svoo_b200 has no CPU or PyTorch fallback")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise ImportError(f"{path} does not export {name}; rebuild it")
        fn.restype = res
        fn.argtypes = args
    if lib.svoo_b200_version() != VERSION:
        raise ImportError(f"{path} is version {lib.svoo_b200_version()}, expected {VERSION}; rebuild it")
    return lib


LIB = _load()


def check(code: int, what: str) -> None:
    """Raise on a non-zero status: ValueError for argument errors, SvooB200Error for CUDA errors."""
    if code == 0:
        return
    msg = LIB.svoo_b200_error_string(code).decode()
    if code < 0:
        raise ValueError(f"{what}: {msg} (status {code})")
    raise SvooB200Error(f"{what}: CUDA error {code}: {msg}")
