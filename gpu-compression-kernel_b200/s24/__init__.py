"""s24 -- B200 (sm_100a) 2:4 structured sparsity: prune, compress, sparse GEMM.

Thin Python layer over libs24.so (C ABI in include/s24.h).  The drop-in modules that
mirror the reference's file and function names live in the sibling `compression`
directory; this package is what they call.
"""
from ._lib import S24Error, lib, LIB_PATH  # noqa: F401
from .ops import (prune, compress, compress_other, prune_compress, meta_convert, meta_tc_numel, spmm,  # noqa: F401
                  spmm_prune_out, spmm_prune_in, spmm_scatter, relayout_shards)
