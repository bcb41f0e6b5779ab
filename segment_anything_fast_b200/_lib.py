"""ctypes binding of ``libsamb200.so`` (the C ABI in ``include/samb200.h``).

There is no fallback: if the library has not been built, or a call returns an
error code, a ``RuntimeError`` is raised.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libsamb200.so")

OK = 0
EPI_BIAS, EPI_GELU, EPI_RESIDUAL, EPI_RAW = 1, 2, 4, 8

_P = c_void_p
# name -> (restype, argtypes); mirrors include/samb200.h one to one.
SIGNATURES = {
    "samb_abi_version": (c_int, []),
    "samb_error_string": (c_char_p, [c_int]),
    "samb_decode_status": (c_int, [c_int32]),
    "samb_selftest_bounded_wait": (c_int, [_P, c_uint32, _P]),
    "samb_selftest_mma_rate": (c_int, [c_int, c_int, c_int, _P, _P, ctypes.POINTER(ctypes.c_double), _P]),
    "samb_layernorm_bf16": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_float, c_int, c_int, _P]),
    "samb_layernorm_quant_i8": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int, c_float, c_int, c_int, _P]),
    "samb_quant_rows_i8": (c_int, [_P, _P, _P, c_int64, c_int, _P]),
    "samb_gelu_quant_rows_i8": (c_int, [_P, _P, _P, c_int64, c_int, _P]),
    "samb_gemm_bf16": (c_int, [_P, c_int64, _P, c_int64, _P, _P, c_int64, c_int64, _P, c_int64, c_int64, c_int,
                               c_int, c_int, _P, _P]),
    "samb_gemm_i8": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, c_int64, c_int64, _P, c_int64, c_int64,
                             c_int, c_int, c_int, _P, _P]),
    "samb_gemm_i8_requant": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, c_int64, _P, _P, _P, c_int64, c_int,
                                     c_int, c_int, _P, _P]),
    "samb_gemm_i8_sp24_requant": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, _P, c_int64, _P, _P, _P, c_int64,
                                          c_int, c_int, c_int, _P, _P]),
    "samb_gemm_i8_requant_static_max_rows": (c_int64, []),
    "samb_gemm_i8_requant_static": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, c_int64, _P, _P, c_int64, c_int,
                                            c_int, c_int, _P, _P]),
    "samb_layernorm2d_nchw": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_float, c_int, _P]),
    "samb_attn_relpos_global": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_attn_relpos_global_f16": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_attn_relpos_global_qkv": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, c_int, c_int, c_int,
                                            c_float, _P, _P]),
    "samb_attn_relpos_global_tables": (c_int, [_P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_attn_relpos_window": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_attn_relpos_window_f16": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_attn_relpos_window_qkv": (c_int, [_P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, c_int, c_int, c_int,
                                            c_int, c_float, _P, _P]),
    "samb_normalize_u8": (c_int, [_P, _P, c_int, c_int, c_int, c_int, ctypes.POINTER(c_float), ctypes.POINTER(c_float), _P]),
    "samb_patch_rows": (c_int, [_P, _P, c_int, c_int, c_int, c_int, _P]),
    "samb_patch_rows_u8": (c_int, [_P, _P, c_int, c_int, c_int, c_int, ctypes.POINTER(c_float), ctypes.POINTER(c_float), _P]),
    "samb_conv3x3_rows": (c_int, [_P, _P, c_int64, c_int, c_int, _P]),
    "samb_relpos_table_products": (c_int, [_P, _P, _P, _P, c_int64, c_int64, c_int, c_int, c_int, _P, _P]),
    "samb_gemm_bf16_heads": (c_int, [_P, c_int64, _P, c_int64, _P, _P, c_int64, c_int, c_int, c_int, _P, _P]),
    "samb_gemm_i8_heads": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, c_int64, c_int, c_int, c_int, _P, _P]),
    "samb_attn_relpos_window_raster": (c_int, [_P, _P, _P, c_int64, c_int, c_int, _P, c_int64, c_int, c_int, c_int, c_int,
                                               c_int, c_float, _P, _P]),
    "samb_attn_relpos_window_tables": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, c_float, _P, _P]),
    "samb_mask_stats": (c_int, [_P, c_int, c_int64, c_int, c_int, c_float, c_float, _P, _P, _P, _P, _P]),
    "samb_mask_rle": (c_int, [_P, c_int64, c_int, c_int, _P, _P, c_int, _P]),
    "samb_sp24_meta_bytes": (c_int64, [c_int, c_int]),
    "samb_pack_sp24": (c_int, [_P, c_int64, c_int, c_int, _P, c_int64, _P, _P, _P]),
    "samb_gemm_i8_sp24": (c_int, [_P, c_int64, _P, _P, c_int64, _P, _P, _P, _P, c_int64, c_int64, _P, c_int64,
                                  c_int64, c_int, c_int, c_int, _P, _P]),
}

_lib = None
_profiler = None


class _Profiled:
    """Forwards every ``samb_*`` call to the library, bracketing it with ``profiler.begin(name, args)``
    / ``profiler.end(token)`` (used by the benchmark to count launches and time kernels with events)."""

    def __init__(self, lib, profiler):
        self._lib, self._profiler = lib, profiler

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        prof = self._profiler

        def call(*args):
            tok = prof.begin(name, args)
            try:
                return fn(*args)
            finally:
                prof.end(tok)
        return call


def set_profiler(profiler):
    """Install (or with ``None`` remove) a launch profiler; see :class:`_Profiled`."""
    global _profiler
    _profiler = profiler


def load():
    """Load the shared library once and attach the declared signatures."""
    global _lib
    if _lib is not None:
        return _lib if _profiler is None else _Profiled(_lib, _profiler)
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the sm_100a kernels are not built "
            "(run `python -m segment_anything_fast_b200.build`). There is no CPU or eager fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def error_string(code):
    return load().samb_error_string(code).decode()


def check(code, what):
    if code != OK:
        raise RuntimeError(f"{what} failed: {error_string(code)} (code {code})")
