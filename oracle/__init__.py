"""CPU oracle for the 2:4 prune / compress / sparse-GEMM path.

TEST INFRASTRUCTURE ONLY: the parity tests, the smoke check and the benchmark's
CPU-baseline leg import this package; the shipped library never does.

The arithmetic lives in ``s24_oracle.c`` (a C restatement of the reference's
``compression/prune.py:57-96`` and ``compression/compress_2_4.py:6-161``); this module
builds it with gcc, loads it with ctypes and wraps it for numpy arrays of raw 16-bit
patterns.  Parity is pinned by the golden vectors in ``tests/golden`` which were
produced by the reference's own Python functions.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "s24_oracle.c"
_LIB = _HERE / "libs24_oracle.so"

FP16, BF16 = 0, 1
MODE_SIGNED, MODE_MAGNITUDE = 0, 1
TIE_REFERENCE, TIE_LOWER, TIE_HIGHER = 0, 1, 2

_lib = None


def build(force: bool = False) -> Path:
    """Compile the C restatement into ``oracle/libs24_oracle.so`` (gcc, OpenMP)."""
    if not force and _LIB.exists() and _LIB.stat().st_mtime >= _SRC.stat().st_mtime:
        return _LIB
    cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-fPIC", "-shared", "-std=c11",
           "-Wall", "-Wextra", "-o", str(_LIB), str(_SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB))
        i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
        L.s24o_prune.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp, vp]
        L.s24o_prune.restype = i32
        L.s24o_prune_f32.argtypes = [vp, i64, i64, i32, i32, vp, vp, vp]
        L.s24o_prune_f32.restype = i32
        L.s24o_compress.argtypes = [vp, i64, i64, i32, vp, vp, vp]
        L.s24o_compress.restype = i32
        L.s24o_compress_other.argtypes = [vp, i64, i64, i32, vp, vp]
        L.s24o_compress_other.restype = i32
        L.s24o_prune_compress.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp, vp, vp]
        L.s24o_prune_compress.restype = i32
        L.s24o_meta_offsets.argtypes = [i64, i64, vp]
        L.s24o_meta_offsets.restype = None
        L.s24o_meta_tc.argtypes = [vp, i64, i64, vp]
        L.s24o_meta_tc.restype = i32
        L.s24o_decompress.argtypes = [vp, vp, i64, i64, vp]
        L.s24o_decompress.restype = None
        L.s24o_gemm_f32acc.argtypes = [vp, vp, i64, i64, i64, i32, vp, vp]
        L.s24o_gemm_f32acc.restype = None
        L.s24o_weak_order_index.argtypes = [vp]
        L.s24o_weak_order_index.restype = i32
        L.s24o_num_threads.restype = i32
        L.s24o_set_num_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def tie_table() -> np.ndarray:
    """729-entry keep-mask table indexed by the weak ordering of a group's four keys.

    Measured from the reference's ``prune_2_4`` (its ``torch.topk`` breaks ties by an
    implementation artefact, not a rule); written by ``tests/golden/make_golden.py``.
    Entries for inconsistent orderings are 0xFF.
    """
    txt = (_HERE / "tie_table.inc").read_text()
    vals = [int(t) for t in txt.replace("\n", " ").split(",") if t.strip()]
    arr = np.array(vals, dtype=np.uint8)
    assert arr.shape == (729,)
    return arr


def _check16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    if a.dtype != np.uint16:
        a = a.view(np.uint16)
    assert a.ndim == 2
    return a


def prune(a_bits: np.ndarray, dtype: int = FP16, mode: int = MODE_SIGNED, tie: int = TIE_REFERENCE,
          return_mask: bool = False):
    """``prune_2_4`` (prune.py:57-96) on raw 16-bit patterns; raises ValueError like :76-77."""
    a = _check16(a_bits)
    M, K = a.shape
    out = np.empty_like(a)
    mask = np.empty((M, max(K // 4, 0)), dtype=np.uint8) if return_mask else None
    tt = tie_table() if tie == TIE_REFERENCE else None
    rc = lib().s24o_prune(_p(a), M, K, dtype, mode, tie, _p(tt), _p(out), _p(mask))
    if rc != 0:
        raise ValueError("The size of the last dimension must be divisible by 4.")
    return (out, mask) if return_mask else out


def prune_f32(a: np.ndarray, mode: int = MODE_SIGNED, tie: int = TIE_LOWER, return_mask: bool = False):
    a = np.ascontiguousarray(a, dtype=np.float32)
    M, K = a.shape
    out = np.empty_like(a)
    mask = np.empty((M, K // 4), dtype=np.uint8) if return_mask else None
    tt = tie_table() if tie == TIE_REFERENCE else None
    rc = lib().s24o_prune_f32(_p(a), M, K, mode, tie, _p(tt), _p(out), _p(mask))
    if rc != 0:
        raise ValueError("The size of the last dimension must be divisible by 4.")
    return (out, mask) if return_mask else out


def compress(dense_bits: np.ndarray, dtype: int = FP16):
    """``compress_dense_to_sparse`` (compress_2_4.py:32-161).

    Returns (vals (M,K/2) uint16, meta_logical (M,K/16) int16, meta_ref (M/16,K) int16).
    Raises RuntimeError for the divisibility conditions the reference rejects.
    """
    d = _check16(dense_bits)
    M, K = d.shape
    if M % 32 != 0:
        raise RuntimeError(f"Number of rows of dense matrix {M} must be divisible by 32")
    if K % 16 != 0:
        raise RuntimeError(f"Number of columns of dense matrix {K} must be divisible by 16")
    if K % 64 != 0:
        raise AssertionError(f"The number of metadata cols must be at least 4, current number: {K // 16}")
    vals = np.empty((M, K // 2), dtype=np.uint16)
    ml = np.empty((M, K // 16), dtype=np.int16)
    mr = np.empty((M // 16, K), dtype=np.int16)
    rc = lib().s24o_compress(_p(d), M, K, dtype, _p(vals), _p(ml), _p(mr))
    assert rc == 0
    return vals, ml, mr


_OTHER_KIND = {np.dtype(np.int8): 0, np.dtype(np.int32): 1, np.dtype(np.float32): 2}


def compress_other(dense: np.ndarray):
    """``compress_dense_to_sparse`` for int8 / int32 / float32 input (compress_2_4.py:41-47,73-76,144-154).

    Returns (vals (M, K/2) of the input type, meta): meta is the reordered buffer viewed
    (M/2, 2 * ncols) like the reference returns it, int32 for int8 input, else int16.
    Raises RuntimeError / AssertionError for the conditions the reference rejects."""
    d = np.ascontiguousarray(dense)
    kind = _OTHER_KIND[d.dtype]
    M, K = d.shape
    rows = 16 if kind == 0 else 32
    cols = 32 if kind == 0 else 16
    if M % rows != 0:
        raise RuntimeError(f"Number of rows of dense matrix {M} must be divisible by {rows}")
    if K % cols != 0:
        raise RuntimeError(f"Number of columns of dense matrix {K} must be divisible by {cols}")
    ncols = K // (32 if kind == 0 else (8 if kind == 2 else 16))
    if ncols % 4 != 0:
        raise AssertionError(f"The number of metadata cols must be at least 4, current number: {ncols}")
    vals = np.empty((M, K // 2), dtype=d.dtype)
    meta = np.empty((M * ncols,), dtype=np.int32 if kind == 0 else np.int16)
    rc = lib().s24o_compress_other(_p(d), M, K, kind, _p(vals), _p(meta))
    assert rc == 0, rc
    return vals, meta.reshape(-1, 2 * ncols)


def prune_compress(a_bits: np.ndarray, dtype: int = FP16, mode: int = MODE_SIGNED, tie: int = TIE_REFERENCE):
    """prune then compress; returns (vals, meta_ref).  Used for the timed CPU baseline."""
    a = _check16(a_bits)
    M, K = a.shape
    scratch = np.empty_like(a)
    vals = np.empty((M, K // 2), dtype=np.uint16)
    mr = np.empty((M // 16, K), dtype=np.int16)
    tt = tie_table() if tie == TIE_REFERENCE else None
    rc = lib().s24o_prune_compress(_p(a), M, K, dtype, mode, tie, _p(tt), _p(scratch), _p(vals), _p(mr))
    if rc != 0:
        raise RuntimeError(f"bad shape ({M}, {K}) for prune+compress (rc={rc})")
    return vals, mr


def meta_offsets(M: int, ncols: int) -> np.ndarray:
    """``_calculate_meta_reordering_offsets`` (compress_2_4.py:6-30)."""
    off = np.empty((M * ncols,), dtype=np.int64)
    lib().s24o_meta_offsets(M, ncols, _p(off))
    return off


def meta_tc(meta_logical: np.ndarray, K: int) -> np.ndarray:
    """Logical metadata -> tcgen05 record layout, uint32 (ceil(M/128) * ceil(K/128) * 512,);
    words of a partly covered last tile / block that lie outside the matrix are 0x44444444."""
    ml = np.ascontiguousarray(meta_logical, dtype=np.int16)
    M = ml.shape[0]
    out = np.empty((-(-M // 128) * -(-K // 128) * 512,), dtype=np.uint32)
    rc = lib().s24o_meta_tc(_p(ml), M, K, _p(out))
    if rc != 0:
        raise RuntimeError("meta_tc needs M % 16 == 0 and K % 64 == 0")
    return out


def decompress(vals: np.ndarray, meta_logical: np.ndarray) -> np.ndarray:
    v = _check16(vals)
    ml = np.ascontiguousarray(meta_logical, dtype=np.int16)
    M, K = v.shape[0], v.shape[1] * 2
    out = np.empty((M, K), dtype=np.uint16)
    lib().s24o_decompress(_p(v), _p(ml), M, K, _p(out))
    return out


def gemm_f32acc(a_bits: np.ndarray, b_bits: np.ndarray, dtype: int = FP16):
    """fp32-accumulated A @ B (gluon_ws_sparse.py:660); returns (C fp32, C rounded bits)."""
    a, b = _check16(a_bits), _check16(b_bits)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c32 = np.empty((M, N), dtype=np.float32)
    c16 = np.empty((M, N), dtype=np.uint16)
    lib().s24o_gemm_f32acc(_p(a), _p(b), M, N, K, dtype, _p(c32), _p(c16))
    return c32, c16


def num_threads() -> int:
    return int(lib().s24o_num_threads())


def set_num_threads(n: int) -> None:
    lib().s24o_set_num_threads(int(n))
