"""Drop-in for compression/kernels/7.8.1_prune_ws.py: sparse GEMM that takes a dense A and
prunes + compresses it inside the kernel (no compressed operand in memory).

The reference keeps this variant as a negative result on Hopper: the prune ran in the warps
that also issue wgmma, on the critical path of every k-step (7.8.1_prune_ws.py:345-374).
Here the prune has warps of its own next to an asynchronous tcgen05 MMA, and dense A goes from
global memory to registers without passing through shared memory.  Every k-block of A is
still pruned once per 480 columns of C, so at large N `run_2_kernel_ws_matmul` stays faster;
at N <= 480 this path reads A once and wins.
"""
import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def run_sparse_ws_matmul(A, B, tune=True, manual_config=None, mode="signed", tie="higher"):
    """C = prune_2_4(A) @ B from the dense A (compression/kernels/7.8.1_prune_ws.py:609-650).

    `tune` and `manual_config` are accepted for signature compatibility; this kernel has one
    tile shape (256 x 480 per CTA pair).  The in-kernel prune ranks signed values with a strict
    compare like the reference's (:122-139), so the higher index survives equal keys.
    """
    return s24.spmm_prune_in(A, B, mode=mode, tie=tie)
