"""ctypes binding of libdqmoe_b200.so (the C ABI declared in include/dqmoe.h).

The library is the only compute path of this package: there is no CPU or
PyTorch fallback. Loading fails loudly when the shared object is missing.
"""
from __future__ import annotations

import ctypes
import os
import re

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# DQMOE_B200_LIB selects another build of the same library (e.g. one compiled with diagnostics)
LIB_PATH = os.environ.get("DQMOE_B200_LIB") or os.path.join(_PKG_DIR, "libdqmoe_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_PKG_DIR), "include", "dqmoe.h")

_c_int = ctypes.c_int
_c_i64 = ctypes.c_int64
_c_size = ctypes.c_size_t
_ptr = ctypes.c_void_p

# name -> (restype, argtypes); must list every function include/dqmoe.h declares
SIGNATURES = {
    "dqmoe_last_error": (ctypes.c_char_p, []),
    "dqmoe_abi_version": (_c_int, []),
    "dqmoe_device_status": (_c_int, [ctypes.POINTER(_c_int)]),
    "dqmoe_moe_workspace_bytes": (_c_size, [_c_int] * 6),
    "dqmoe_moe_forward": (_c_int, [_ptr] * 9 + [_c_size] + [_c_int] * 7 + [_ptr]),
    "dqmoe_moe_workspace_ptr": (_ptr, [_ptr] + [_c_int] * 7),
    "dqmoe_moe_forward_f16": (_c_int, [_ptr] * 6 + [_c_size] + [_c_int] * 5 + [_ptr]),
    "dqmoe_moe_forward_bias": (_c_int, [_ptr] * 11 + [_c_size] + [_c_int] * 6 + [_ptr]),
    "dqmoe_moe_forward_f16_bias": (_c_int, [_ptr] * 8 + [_c_size] + [_c_int] * 5 + [_ptr]),
    "dqmoe_moe_workspace_bytes_f32": (_c_size, [_c_int] * 5),
    "dqmoe_moe_forward_f32": (_c_int, [_ptr] * 8 + [_c_size] + [_c_int] * 5 + [_ptr]),
    "dqmoe_moe_block_workspace_bytes": (_c_size, [_c_int] * 6),
    "dqmoe_moe_block": (_c_int, [_ptr] * 8 + [_c_size] + [_c_int] * 7 + [_ptr]),
    "dqmoe_moe_block_shared": (_c_int, [_ptr] * 8 + [_c_size] + [_c_int] * 8 + [_ptr]),
    "dqmoe_route_topk": (_c_int, [_ptr, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_route_sort_workspace_bytes": (_c_size, [_c_int, _c_int]),
    "dqmoe_route_sort": (_c_int, [_ptr, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_size, _ptr]),
    "dqmoe_segment_ids": (_c_int, [_ptr, _ptr, _c_int, _ptr, _c_int, _ptr]),
    "dqmoe_permute_rows": (_c_int, [_ptr, _c_size, _c_int, _ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr]),
    "dqmoe_permute_quant_block_1x128": (_c_int, [_ptr, _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_finalize_scatter": (_c_int, [_ptr, _c_size, _ptr, _c_int, _ptr, _ptr]),
    "dqmoe_finalize_weighted": (_c_int, [_ptr, _ptr, _ptr, _c_int, _c_int, _c_int, _ptr]),
    "dqmoe_quant_fp8_rowwise": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_quant_fp8_block_1x128": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_quant_fp8_block_128x128": (_c_int, [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_quant_fp8_tensor": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr]),
    "dqmoe_quant_fp8_tensor_static": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _ptr]),
    "dqmoe_quant_mxfp8": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_permute_quant_mxfp8": (_c_int, [_ptr, _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_mx_tiled_scale_bytes": (_c_size, [_c_i64, _c_int, _c_int]),
    "dqmoe_mx_tile_scales": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr]),
    "dqmoe_grouped_gemm_mx": (_c_int, [_ptr] * 6 + [_c_int] * 5 + [_ptr] * 4),
    "dqmoe_grouped_gemm_mx_rows": (_c_int, [_ptr] * 6 + [_c_int] * 4 + [_ptr, _ptr]),
    "dqmoe_quant_nvfp4": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr]),
    "dqmoe_grouped_gemm_nvfp4": (_c_int, [_ptr] * 8 + [_c_int] * 5 + [_ptr] * 5),
    "dqmoe_moe_forward_nvfp4": (_c_int, [_ptr] * 15 + [_c_size] + [_c_int] * 5 + [_ptr]),
    "dqmoe_grouped_gemm": (_c_int, [_ptr] * 6 + [_c_int] * 6 + [_ptr] * 5),
    "dqmoe_grouped_gemm_rows": (_c_int, [_ptr] * 6 + [_c_int] * 5 + [_ptr, _ptr]),
    "dqmoe_ep_publish_counts": (_c_int, [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _ptr]),
    "dqmoe_ep_plan": (_c_int, [_ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr]),
    "dqmoe_ep_set_wait_limit": (_c_int, [_c_i64]),
    "dqmoe_ep_publish_plan": (_c_int, [_ptr, _c_int, _c_int, _c_int, _ptr, _ptr, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr]),
    "dqmoe_ep_signal_wait": (_c_int, [_ptr, _c_int, _c_int, _c_int, _c_int, _ptr]),
    "dqmoe_ep_dispatch": (_c_int, [_ptr, _ptr, _c_size, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _c_int, _c_int,
                                   _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr]),
    "dqmoe_ep_wait": (_c_int, [_ptr, _c_int, _c_int, _c_int, _ptr]),
    "dqmoe_ep_signal": (_c_int, [_ptr, _c_int, _c_int, _c_int, _c_int, _ptr]),
    "dqmoe_ep_row_ptrs": (_c_int, [_ptr, _ptr, _c_int, _ptr, _c_int, _c_size, _c_int, _ptr, _ptr]),
    "dqmoe_ep_wait_row_ptrs": (_c_int, [_ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _c_int, _c_size, _c_int, _ptr, _ptr]),
    "dqmoe_mtile_prefix": (_c_int, [_ptr, _c_int, _ptr, _ptr]),
    "dqmoe_requant_from_amax": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr]),
    "dqmoe_requant_from_amax_dev": (_c_int, [_ptr, _c_i64, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr]),
    "dqmoe_plugin_create": (_c_int, [_ptr, ctypes.POINTER(_ptr)]),
    "dqmoe_plugin_destroy": (None, [_ptr]),
    "dqmoe_plugin_get_fields": (_c_int, [_ptr, _ptr]),
    "dqmoe_plugin_workspace_size": (_c_size, [_ptr, _c_int]),
    "dqmoe_plugin_enqueue": (_c_int, [_ptr, _c_int, _ptr, _ptr, _ptr, _ptr]),
    "dqmoe_plugin_serialization_size": (_c_size, []),
    "dqmoe_plugin_serialize": (_c_int, [_ptr, _ptr, _c_size]),
    "dqmoe_plugin_deserialize": (_c_int, [_ptr, _c_size, ctypes.POINTER(_ptr)]),
}

_lib = None


def declared_symbols(header_path: str = HEADER_PATH):
    """Names of all functions declared in include/dqmoe.h."""
    with open(header_path) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dqmoe_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    """Load the native library (once) and set the ctypes signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m dqmoe_b200.build` "
            "(dqmoe_b200 has no fallback path without its CUDA library)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.dqmoe_abi_version() != 1:
        raise RuntimeError("libdqmoe_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def check(rc: int) -> None:
    """Turn a non-zero return code into RuntimeError carrying the library's message."""
    if rc != 0:
        msg = load().dqmoe_last_error().decode("utf-8", "replace")
        raise RuntimeError(msg or f"dqmoe_b200 call failed with code {rc}")
