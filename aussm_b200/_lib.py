"""ctypes binding of libaussm_b200.so (declared in include/aussm_b200.h).

The library is the product: there is no Python or CPU fallback.  If it has
not been built, importing the operators fails with instructions.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libaussm_b200.so")

_P = ctypes.c_void_p
_I = ctypes.c_int
_Z = ctypes.c_size_t
_LL = ctypes.c_longlong

# name -> (restype, argtypes); mirrors include/aussm_b200.h one to one
SIGNATURES = {
    "aussm_b200_version": (_I, []),
    "aussm_b200_last_error": (ctypes.c_char_p, []),
    "aussm_b200_device_status": (_I, [_P]),
    "aussm_b200_set_option": (_I, [ctypes.c_char_p, _I]),
    "aussm_b200_scan_unitary_fwd": (_I, [_P] * 14 + [_I] * 4 + [_P]),
    "aussm_b200_scan_unitary_fwd_workspace_bytes": (_Z, [_I] * 4),
    "aussm_b200_scan_unitary_fwd_ws": (_I, [_P] * 14 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_scan_unitary_bwd_workspace_bytes": (_Z, [_I] * 4),
    "aussm_b200_scan_unitary_bwd": (_I, [_P] * 25 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_scan_unitary_bwd_static": (_I, [_P] * 25 + [_I] * 4 + [_P]),
    "aussm_b200_kernel_launches": (ctypes.c_ulonglong, []),
    "aussm_b200_gemm_split3_workspace_bytes": (_Z, [_I] * 8),
    "aussm_b200_gemm_split3": (_I, [_P, _I, _I, _P, _I, _I, _P] + [_I] * 6 + [_P, _Z, _P]),
    "aussm_b200_gemm_split3_strided": (_I, [_P, _I, _LL, _LL, _P, _I, _LL, _LL, _P, _LL, _LL] + [_I] * 6 + [_P, _Z, _P]),
    "aussm_b200_unitary_workspace_bytes": (_Z, [_I] * 4),
    "aussm_b200_scan_complex_states_floats": (_Z, [_I] * 4),
    "aussm_b200_scan_complex_bwd_workspace_bytes": (_Z, [_I] * 4),
    "aussm_b200_scan_complex_fwd": (_I, [_P] * 12 + [_I] * 4 + [_P]),
    "aussm_b200_scan_complex_bwd": (_I, [_P] * 23 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_complex_workspace_bytes": (_Z, [_I] * 5),
    "aussm_b200_complex_fwd": (_I, [_P] * 3 + [_I] + [_P] * 8 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_complex_bwd": (_I, [_P] * 5 + [_I] + [_P] * 16 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_selective_scan_ckpt_floats": (_Z, [_I] * 4),
    "aussm_b200_selective_scan_bwd_workspace_bytes": (_Z, [_I] * 4),
    "aussm_b200_selective_scan_fwd": (_I, [_P] * 8 + [_I] + [_P] * 3 + [_I] * 4 + [_P]),
    "aussm_b200_selective_scan_bwd": (_I, [_P] * 9 + [_I] + [_P] * 9 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_conv_pre_fwd": (_I, [_P] * 4 + [_I] * 4 + [_P]),
    "aussm_b200_conv_pre_bwd_workspace_bytes": (_Z, [_I] * 2),
    "aussm_b200_conv_pre_bwd": (_I, [_P] * 6 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_softplus_bias_fwd": (_I, [_P, _P, ctypes.c_float, _P] + [_I] * 3 + [_P]),
    "aussm_b200_softplus_bias_bwd_workspace_bytes": (_Z, [_I] * 2),
    "aussm_b200_softplus_bias_bwd": (_I, [_P, _P, ctypes.c_float, _P, _P] + [_I] * 3 + [_P, _Z, _P]),
    "aussm_b200_unitary_fwd": (_I, [_P] * 15 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_unitary_bwd": (_I, [_P] * 29 + [_I] * 4 + [_P, _Z, _P]),
    "aussm_b200_unitary_keep_bytes": (_Z, [_I] * 4),
    "aussm_b200_unitary_fwd_keep": (_I, [_P] * 15 + [_I] * 4 + [_P, _Z, _P, _Z, _P]),
    "aussm_b200_unitary_bwd_kept": (_I, [_P] * 29 + [_I] * 4 + [_P, _Z, _P, _Z, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m aussm_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback implementation.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().aussm_b200_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def set_option(name: str, value: int) -> None:
    check(load().aussm_b200_set_option(name.encode(), int(value)), f"set_option({name})")
