"""Drop-in for the reference's compression/compress_2_4.py.

`compress_dense_to_sparse` keeps the reference's signature, return shapes, metadata
layout and error behaviour and runs on the B200 through libs24 (C ABI `s24_compress` for
fp16 / bf16, the types the sparse GEMM consumes; `s24_compress_other` for the int8, int32 and
float32 branches).
"""
import torch

import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def _calculate_meta_reordering_offsets(m, meta_ncols, device):
    """Destination of logical metadata word (row, col) in the reordered buffer
    (compression/compress_2_4.py:6-30): rows interleave in pairs (r, r+8) inside blocks of
    16 rows x 4 words."""
    assert meta_ncols % 4 == 0, f"The number of metadata cols must be at least 4, current number: {meta_ncols}"
    row = torch.arange(m, device=device, dtype=torch.int64).unsqueeze(1)
    col = torch.arange(meta_ncols, device=device, dtype=torch.int64).unsqueeze(0)
    dst_col = (col // 4) * 64 + (row % 8) * 8 + (row // 8) % 2 + (col % 4) * 2
    return ((row // 16) * (meta_ncols * 16) + dst_col).reshape(-1)


def compress_dense_to_sparse(dense):
    """(values (m, k/2), metadata int16 viewed (m/2, k/8)) from the non-zero pattern of
    `dense` (compression/compress_2_4.py:32-161).  Callers re-view the metadata as
    (m/16, k) (compression/gluon_ws_sparse.py:656)."""
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    if dense.dtype in (torch.int8, torch.float, torch.int32):   # compress_2_4.py:41-47,73-76,144-154
        return s24.compress_other(dense)
    if dense.dtype not in (torch.half, torch.bfloat16):
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    m, k = dense.shape
    if m % 32 != 0:
        raise RuntimeError(f"Number of rows of dense matrix {m} must be divisible by 32")
    if k % 16 != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by 16")
    if m * k == 0:
        return dense, torch.zeros(dense.shape, dtype=torch.int16, device=dense.device)
    vals, e, _ = s24.compress(dense, want_ref=True, want_tc=False)
    return vals, e.view(-1, k // 8)
