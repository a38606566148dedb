"""Drop-in for compression/dev/10.2_prune_acc_2_kernel.py: the "separated" comparison line of
the fused-output experiment -- sparse GEMM to a dense C, then the standalone prune+compress
kernel applied to C along N.
"""
import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def _tiles(cfg):
    if not cfg:
        return None
    return {k: cfg[k] for k in ("BM", "BN") if cfg.get(k) in (128, 224, 256, 512)} or None


def run_matmul_then_compress_separate(A_comp, E_A, B, tune=True, manual_matmul_config=None,
                                      manual_compress_config=None):
    """(C_dense, C_vals, C_meta) as compression/dev/10.2_prune_acc_2_kernel.py:561-650 returns
    them.  The second kernel ranks the rounded 16-bit C with strict `>` like the reference's
    (ties keep the higher index); `manual_compress_config` has no meaning here and is ignored."""
    C = s24.spmm(A_comp, E_A, B, meta_layout="ref", manual_config=None if tune else _tiles(manual_matmul_config))
    c_vals, c_meta, _ = s24.prune_compress(C, mode="signed", tie="higher", want_ref=True, want_tc=False)
    return C, c_vals, c_meta
