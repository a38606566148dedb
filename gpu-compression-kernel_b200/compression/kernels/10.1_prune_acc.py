"""Drop-in for compression/kernels/10.1_prune_acc.py: sparse GEMM whose epilogue 2:4-prunes
the fp32 accumulator along N and stores it already compressed.

`run_sparse_ws_matmul(A, E, B, tune=True, manual_config=None)` keeps the reference's
arguments and returns `(C_vals, C_meta)`: values (M, N/2) in A's dtype and metadata
(M/16, N) int16 in the reference's reordered layout (10.1_prune_acc.py:624-678).
"""
import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def run_sparse_ws_matmul(A, E, B, tune=True, manual_config=None):
    """(C_vals, C_meta) = compress(prune_2_4(A24 @ B)) with the pruning done in the GEMM's epilogue
    (signed keys, the lower index survives a tie: 10.1_prune_acc.py:100-105).  The accumulators are
    rounded to the output type first and ranked then, so the result equals prune + compress of the
    dense product the plain launcher returns; the reference ranks the fp32 values and rounds the
    survivors (:241), which differs only where two sums of a group round to the same number."""
    cfg = None
    if not tune and manual_config:
        cfg = {k: manual_config[k] for k in ("BM", "BN") if manual_config.get(k) in (128, 224, 256, 512)} or None
    c_vals, c_meta, _ = s24.spmm_prune_out(A, E, B, meta_layout="ref", want_ref=True, want_tc=False, manual_config=cfg)
    return c_vals, c_meta


def run_sparse_ws_matmul_chained(A, meta_tc, B, manual_config=None):
    """Same product with metadata in and out in the tensor-core layout, so that the result
    can be the sparse operand of a following GEMM without any re-layout."""
    c_vals, _, c_tc = s24.spmm_prune_out(A, meta_tc, B, meta_layout="tc", want_ref=False, want_tc=True,
                                         manual_config=manual_config)
    return c_vals, c_tc
