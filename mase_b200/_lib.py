"""ctypes binding of libmxq.so, the C-ABI library declared in include/mxq.h.

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_void_p, c_char_p

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libmxq.so")
_lib = None

# name -> argument types, exactly the prototypes of include/mxq.h
_PROTOTYPES = {
    "mxq_version": [],
    "mxq_mxint_fake": [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxint_extract": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxint_compose": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p],
    "mxq_mxint_clip_search": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxfp_clip_search": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_int,
                             c_void_p, c_void_p],
    "mxq_mxfp_fake": [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxfp_extract": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxfp_compose": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p],
    "mxq_minifloat_fake": [c_void_p, c_void_p, c_int, c_int, c_int64, c_int, c_int, c_void_p],
    "mxq_gemm_dense": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int64, c_void_p,
                       c_void_p, c_void_p],
    "mxq_gemm_dense_batched": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64,
                               c_int64, c_int64, c_void_p, c_void_p, c_void_p],
    "mxq_mma_scale_bytes": [c_int64, c_int64],
    "mxq_gemm_options_size": [],
    "mxq_mxfp_pack_mma": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p],
    "mxq_mxfp4_pack_mma": [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p],
    "mxq_gemm_mxf8": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
                      c_int64, c_void_p, c_void_p, c_void_p],
    "mxq_mx_linear_workspace_bytes": [c_int64, c_int64],
    "mxq_mx_linear": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64,
                      c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p],
    "mxq_silu_mul_pack_mma": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p,
                              c_void_p],
    "mxq_mx_gated_linear": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64,
                            c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p],
    "mxq_attention_softmax": [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, ctypes.c_float, c_void_p, c_int64, c_int64,
                              c_int64, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mxq_softmax_quant": [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "mxq_rope": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_int64,
                 c_int64, c_int64, c_int64, c_void_p],
    "mxq_gemm_mxf8_scatter": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int64, c_int64,
                              c_int64, c_void_p, c_void_p, c_void_p],
    "mxq_peer_barrier": [c_void_p, c_int, c_int, ctypes.c_uint32, c_void_p, c_int64, c_void_p],
    "mxq_reduce_gather": [c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "mxq_reduce_gather_pack": [c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                               c_int, c_void_p, c_int, c_void_p],
    "mxq_mx_linear_static": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
                             c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "mxq_bfp_fake_tiles": [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                           c_void_p, c_void_p],
    "mxq_bfp_fake": [c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
}


class GemmOptions(ctypes.Structure):
    """`mxq_gemm_options` of include/mxq.h: per-call settings of the GEMM entry points (all zero = defaults)."""

    _fields_ = [("max_ctas", ctypes.c_int32), ("tiles", ctypes.c_int32), ("no_split_k", ctypes.c_int32),
                ("flags", ctypes.c_int32), ("wait_limit_ns", ctypes.c_int64), ("test_hook", ctypes.c_int32),
                ("no_transposed", ctypes.c_int32)]


TILES_AUTO, TILES_SINGLE, TILES_PAIRS = 0, 1, 2
GEMM_STATIC_B, GEMM_A_E5M2 = 1, 4  # bits of GemmOptions.flags
CODES_E4M3, CODES_E2M1X2, CODES_E5M2 = 0, 1, 2
TEST_DROP_LAST_LOAD = 1


class MxqError(RuntimeError):
    pass


def library_path() -> str:
    return _PATH


def exported_symbols() -> list[str]:
    return sorted(_PROTOTYPES) + ["mxq_error_string"]


def lib():
    """The loaded library.  Raises if it has not been built (`python -m mase_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            raise MxqError(
                f"{_PATH} is missing: build it with `python -m mase_b200.build` (needs nvcc). "
                "mase_b200 has no CPU or eager fallback."
            )
        handle = ctypes.CDLL(_PATH)
        for name, argtypes in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = c_int64 if name.endswith("_bytes") else c_int
        handle.mxq_error_string.argtypes = [c_int]
        handle.mxq_error_string.restype = c_char_p
        if handle.mxq_gemm_options_size() != ctypes.sizeof(GemmOptions):
            raise MxqError("mxq_gemm_options of libmxq.so and its ctypes mirror differ in size: rebuild the library")
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().mxq_error_string(code).decode()
        raise MxqError(f"{what} failed: {msg} (code {code})")
