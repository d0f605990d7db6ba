"""ctypes binding of libbsp_b200.so (the C ABI declared in include/bsp.h).

The library is the only compute path of this package: there is no Python or
CPU fallback.  If the shared object is missing it is compiled on first use
(needs nvcc); if that fails the import error is raised to the caller.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

from . import _build

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CAPACITY, ERR_CUDA, ERR_EMPTY_HEAD, ERR_TIMEOUT = range(7)
F32, F16, BF16 = 0, 1, 2
MAX_PACKS = 8
META_HEADER = 8
ATTN_STATIC_ROWS = 1 << 20

_lib = None

_I64P = POINTER(c_int64)
_I32P = POINTER(c_int32)
_IP = POINTER(c_int)
_STRIDE3 = [c_int64, c_int64, c_int64]
_MASKS = [c_void_p] + _STRIDE3 + [c_void_p, c_int64, c_int, c_void_p, c_int64, c_int]

_SIGNATURES = {
    'bsp_last_error': (c_char_p, []),
    'bsp_abi_version': (c_int, []),
    'bsp_sdd_lut_build': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                  _I32P, _I64P, _I64P, _IP, _I64P]),
    'bsp_dxx_lut_build': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_void_p, c_int64, _I64P, _IP, _IP]),
    'bsp_softmax_lut_build': (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int64, _I64P, _IP]),
    'bsp_softmax_lut_from_meta': (c_int, [c_void_p, c_void_p, c_void_p, c_int64, _I64P, _IP, c_void_p]),
    'bsp_fixed_layout_build': (c_int, [c_int] * 7 + [c_void_p]),
    'bsp_window_layout_build': (c_int, [c_int] * 6 + [c_void_p, c_int, c_void_p]),
    'bsp_device_status': (c_int, [_IP]),
    'bsp_debug_attn_wait': (c_int, [c_int, c_int]),
    'bsp_matmul_use_tcgen05': (c_int, [c_int]),
    'bsp_attn_tiles_build': (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int64, _I64P]),
    'bsp_meta_build': (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int64, _I64P]),
    'bsp_attn_tiles_device_capacity': (c_int64, [c_int, c_int, c_int]),
    'bsp_attn_tiles_build_device': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    'bsp_meta_validate': (c_int, [c_void_p, c_int64, _IP, _IP, c_void_p]),
    'bsp_attn_tiles_validate': (c_int, [c_void_p, c_int64, _IP, _IP, c_void_p]),
    'bsp_meta_device_capacity': (c_int64, [c_int, c_int, c_int]),
    'bsp_meta_build_device': (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    'bsp_softmax_fwd': (c_int, [c_void_p, c_int, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_int, c_float]
                        + _MASKS + [c_void_p]),
    'bsp_softmax_bwd': (c_int, [c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int, c_int, c_int,
                                c_void_p, c_int, c_float, c_void_p]),
    'bsp_sdd': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]
                + [c_int64] * 9 + [c_void_p, c_void_p, c_void_p]),
    'bsp_dsd': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64, c_int]
                + [c_int64] * 8 + [c_void_p, c_void_p, c_void_p]),
    'bsp_dds': (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]
                + [c_int64] * 4 + [c_int64, c_int] + [c_int64] * 4 + [c_void_p, c_void_p, c_void_p]),
    'bsp_attn_fwd': (c_int, [c_void_p] * 5 + [c_int] * 6 + [c_int64] * 12 + [c_void_p] * 4 + [c_float]
                     + _MASKS + [c_void_p]),
    'bsp_attn_bwd': (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_int64] * 15 + [c_void_p] * 4 + [c_float]
                     + _MASKS + [c_void_p]),
    'bsp_attn_bwd_static': (c_int, [c_void_p] * 9 + [c_int] * 6 + [c_int64] * 15 + [c_void_p] * 4 + [c_float]
                            + _MASKS + [c_void_p]),
    'bsp_attn_bwd_parts': (c_int, [c_void_p] * 10 + [c_int] * 6 + [c_int64] * 15 + [c_void_p] * 4 + [c_float]
                           + _MASKS + [c_int, c_void_p]),
}


def exported_symbols():
    """Names every build of the library must export (one per declaration in include/bsp.h)."""
    return sorted(_SIGNATURES)


def lib():
    """Loads (building first if necessary) and returns the ctypes library handle."""
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path) or (os.environ.get('BSP_REBUILD') and _build.needs_build()):
            path = _build.build()
        handle = ctypes.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue   # reported by the symbol test; calling it raises AttributeError
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


_EXC = {ERR_INVALID: ValueError, ERR_UNSUPPORTED: NotImplementedError, ERR_CAPACITY: RuntimeError,
        ERR_CUDA: RuntimeError, ERR_EMPTY_HEAD: RuntimeError, ERR_TIMEOUT: RuntimeError}


def device_status():
    """Reads and clears the device status words (synchronises): 0, or the code of the tcgen05
    kernel family in which a bounded wait expired."""
    out = c_int(0)
    rc = lib().bsp_device_status(ctypes.byref(out))
    if rc not in (OK, ERR_TIMEOUT):
        check(rc)
    return out.value


def check_device():
    """Raises RuntimeError when a bounded device-side wait has expired since the last check."""
    out = c_int(0)
    check(lib().bsp_device_status(ctypes.byref(out)))


def check(status):
    """Raises the Python exception that corresponds to a non-zero C status."""
    if status != OK:
        msg = lib().bsp_last_error().decode('utf-8', 'replace')
        raise _EXC.get(status, RuntimeError)(msg)
