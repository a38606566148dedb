"""Drop-in for the launcher of the reference's compression/gluon_ws_sparse.py.

`run_sparse_ws_matmul(A, E, B, tune=True, manual_config=None)` keeps the reference's
arguments: A = compressed values (M, K/2), E = the reference-layout metadata (M/16, K)
int16, B = (K, N) row-major; returns a freshly allocated C (M, N).  The work is done by
the tcgen05 kernel behind `s24_spmm_ref_meta`; the metadata is re-laid for the tensor core
into a scratch tensor on every call (a few microseconds).
"""
import warnings

import torch

import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402

_KNOWN_KEYS = {"BM", "BN", "BK", "warps", "buffers", "SF"}


def _normalise_config(manual_config):
    """Map the reference's manual_config keys (gluon_ws_sparse.py:629-636) onto the tile
    variants this library has; keys with no meaning here (BK, warps, SF) are ignored."""
    if not manual_config:
        return None
    unknown = set(manual_config) - _KNOWN_KEYS
    if unknown:
        warnings.warn(f"ignoring unknown manual_config keys {sorted(unknown)}")
    cfg = {}
    bm, bn = manual_config.get("BM"), manual_config.get("BN")
    if bm in (128, 256, 512):
        cfg["BM"] = bm
    if bn in (128, 224, 256):
        cfg["BN"] = bn
    return cfg or None


def run_sparse_ws_matmul(A, E, B, tune=True, manual_config=None):
    """C = A24 @ B (compression/gluon_ws_sparse.py:560-613); fp32 accumulate, C in A's dtype.

    `tune=True` times the library's tile shapes once per (M, N, K) and keeps the fastest (the
    reference autotunes over its Triton configs the same way, :528-535,572-582); with
    `tune=False` the BM / BN entries of `manual_config` are honoured, or the built-in
    heuristic if there are none.
    """
    if tune:
        return s24.spmm(A, E, B, meta_layout="ref", autotune=True)
    return s24.spmm(A, E, B, meta_layout="ref", manual_config=_normalise_config(manual_config))
