"""Drop-in for compression/kernels/11.1_2_kernel_baseline.py: dense A -> fused
prune+compress kernel -> sparse GEMM, two launches on one stream.

The metadata goes from the first kernel to the second in the tensor-core layout, so no
re-layout runs in between (the property the reference gets from emitting its reordered E
directly, 11.1_2_kernel_baseline.py:120-122,288-296).
"""
import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def run_2_kernel_ws_matmul(A, B, tune=True, manual_config=None, mode="signed", tie="higher"):
    """C = prune_2_4(A) @ B (compression/kernels/11.1_2_kernel_baseline.py:256-349).

    The reference's fused kernel compares with strict `>` so the higher index survives a
    tie (:95-100); that is the default here.  Pass tie="reference" for the behaviour of
    the torch `prune_2_4`.
    """
    vals, _, meta_tc = s24.prune_compress(A, mode=mode, tie=tie, want_ref=False, want_tc=True)
    cfg = None
    if not tune and manual_config:
        cfg = {k: manual_config[k] for k in ("BM", "BN") if manual_config.get(k) in (128, 224, 256, 512)} or None
    return s24.spmm(vals, meta_tc, B, meta_layout="tc", manual_config=cfg)


def run_compress(A, mode="signed", tie="higher"):
    """The first launch alone: (values, E in the reference layout)."""
    vals, e, _ = s24.prune_compress(A, mode=mode, tie=tie, want_ref=True, want_tc=False)
    return vals, e
