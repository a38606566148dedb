"""ctypes binding of libs24.so (declarations follow include/s24.h one for one)."""
from __future__ import annotations

import ctypes
from pathlib import Path

import os

_HERE = Path(__file__).resolve().parent
# S24_LIBRARY=<path> loads another build of the library (a variant made with build.py --define ... --out ...)
LIB_PATH = Path(os.environ["S24_LIBRARY"]) if os.environ.get("S24_LIBRARY") else _HERE / "libs24.so"

OK = 0
ERR_INVALID_ARG, ERR_SHAPE, ERR_CUDA, ERR_UNSUPPORTED, ERR_TIMEOUT = -1, -2, -3, -4, -5
FP16, BF16 = 0, 1
INT8, INT32, FP32 = 2, 3, 4
MODE_SIGNED, MODE_MAGNITUDE = 0, 1
TIE_REFERENCE, TIE_LOWER, TIE_HIGHER = 0, 1, 2
META_LOGICAL, META_REF, META_TC = 0, 1, 2
STATIC_SCRATCH_BYTES = 8 << 20
PEER_HANDLE_BYTES = 64

# every symbol include/s24.h declares, with (restype, argtypes)
_vp, _i64, _i32, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t


class TileCfg(ctypes.Structure):
    _fields_ = [("bm", _i32), ("bn", _i32), ("stages", _i32), ("reserved", _i32)]


SIGNATURES = {
    "s24_version": (_i32, []),
    "s24_last_error": (ctypes.c_char_p, []),
    "s24_prune": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp]),
    "s24_compress": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp, _vp]),
    "s24_compress_other": (_i32, [_vp, _i64, _i64, _i64, _i32, _vp, _vp, _vp]),
    "s24_prune_compress": (_i32, [_vp, _i64, _i64, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "s24_meta_tc_bytes": (_sz, [_i64, _i64]),
    "s24_meta_convert": (_i32, [_vp, _i32, _vp, _i32, _i64, _i64, _vp]),
    "s24_spmm": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, ctypes.POINTER(TileCfg), _vp]),
    "s24_spmm_bt": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, ctypes.POINTER(TileCfg), _vp]),
    "s24_spmm_ref_meta": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32,
                                 ctypes.POINTER(TileCfg), _vp, _sz, _vp]),
    "s24_spmm_ref_meta_noalloc": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32,
                                         ctypes.POINTER(TileCfg), _vp]),
    "s24_spmm_prune_out": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32,
                                  ctypes.POINTER(TileCfg), _vp]),
    "s24_spmm_prune_in": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "s24_spmm_scatter": (_i32, [_vp, _vp, _vp, ctypes.POINTER(_vp), _i32, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "s24_peer_alloc": (_i32, [_sz, ctypes.POINTER(_vp)]),
    "s24_peer_free": (_i32, [_vp]),
    "s24_peer_export": (_i32, [_vp, _vp]),
    "s24_peer_open": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "s24_peer_close": (_i32, [_vp]),
    "s24_peer_copy_2d": (_i32, [_vp, _sz, _vp, _sz, _sz, _sz, _vp]),
    "s24_relayout_shards": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "s24_device_status": (_i32, [_vp]),
    "s24_selftest_timeout": (_i32, [_i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, ctypes.POINTER(TileCfg), _vp]),
}

_lib = None


class S24Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libs24 error {code}: {text}")
        self.code = code
        self.text = text


def lib() -> ctypes.CDLL:
    """Load the CUDA library.  There is no fallback: a missing build is an error."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python gpu-compression-kernel_b200/build.py` "
                "(there is no CPU or PyTorch fallback for these kernels)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().s24_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != OK:
        raise S24Error(code, last_error())
