"""The allocation-free GEMM entry point, s24_spmm_ref_meta_noalloc, through the C ABI.

Some users of the library cannot allocate device memory when they call it: their HBM budget
was fixed when their process started (a serving plugin, an embedded host with its own
allocator) or they sit in a loop that cannot take cudaMalloc's synchronisation.  For them the
library keeps the metadata scratch buffer inside its own image.  This test calls that entry
point with caller-owned inputs and outputs only and checks that it gives exactly what
s24_spmm_ref_meta gives with a caller-provided workspace -- twice in a row with different
problems, because the built-in buffer is shared and still holds the previous call's bytes.
It also checks that a problem too large for the built-in buffer is refused with a clear
message.  The file name sorts last so that a run stopping at the first failure has already
run every other test; the test does not depend on anything the other tests did.
"""
import ctypes

import numpy as np
import pytest
import torch

from util import bits, from_bits, oracle, randn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _problem(M, K, N, dtype, seed):
    A = randn((M, K), dtype, seed)
    B = randn((K, N), dtype, seed + 1).to(DEV)
    ap = oracle.prune(bits(A), oracle.FP16 if dtype == torch.float16 else oracle.BF16)
    vals, ml, e = oracle.compress(ap, oracle.FP16 if dtype == torch.float16 else oracle.BF16)
    return from_bits(vals, dtype, DEV), torch.from_numpy(e).to(DEV), B, ap


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row():
    from s24 import _lib
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    torch.backends.cuda.matmul.allow_tf32 = False
    with torch.cuda.device(DEV):
        # the third problem covers its last 128 x 128 metadata records only partly: the conversion into the
        # built-in buffer must also give the words outside the matrix a valid code
        for call, (M, K, N, dtype) in enumerate([(512, 1024, 768, torch.float16), (256, 384, 1032, torch.bfloat16),
                                                 (160, 192, 72, torch.float16)]):
            vals, E, B, ap = _problem(M, K, N, dtype, 900 + call)
            dt = _lib.FP16 if dtype == torch.float16 else _lib.BF16
            # existing entry point: caller-provided workspace
            ws = torch.empty(int(L.s24_meta_tc_bytes(M, K)) // 4, dtype=torch.int32, device=DEV)
            C_ws = torch.empty(M, N, dtype=dtype, device=DEV)
            _lib.check(L.s24_spmm_ref_meta(_vp(vals), _vp(E), _vp(B), _vp(C_ws), M, N, K, N, N, dt, None,
                                           _vp(ws), ws.numel() * 4, stream))
            # new entry point: inputs and outputs only
            C_na = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
            _lib.check(L.s24_spmm_ref_meta_noalloc(_vp(vals), _vp(E), _vp(B), _vp(C_na), M, N, K, N, N, dt, None, stream))
            torch.cuda.synchronize()
            assert L.s24_device_status(None) == 0, _lib.last_error()
            # same kernel, same operands: identical bits; and right within the GEMM tolerance
            assert torch.equal(C_na, C_ws), f"call {call}: no-alloc result differs from the workspace entry point"
            ref = from_bits(ap, dtype, DEV).float() @ B.float()
            torch.testing.assert_close(C_na.float(), ref, rtol=1e-2, atol=1e-2 + 8e-3 * float(ref.abs().max()))


def test_noalloc_entry_accepts_a_problem_that_fills_its_buffer_exactly():
    """8192 x 8192: s24_meta_tc_bytes = 8 MiB = the whole built-in buffer"""
    from s24 import _lib
    L = _lib.lib()
    M = K = 8192
    N = 128
    assert int(L.s24_meta_tc_bytes(M, K)) == _lib.STATIC_SCRATCH_BYTES
    stream = ctypes.c_void_p(torch.cuda.current_stream(torch.device(DEV)).cuda_stream)
    with torch.cuda.device(DEV):
        vals, E, B, ap = _problem(M, K, N, torch.float16, 8192)
        ws = torch.empty(_lib.STATIC_SCRATCH_BYTES // 4, dtype=torch.int32, device=DEV)
        C_ws = torch.empty(M, N, dtype=torch.float16, device=DEV)
        _lib.check(L.s24_spmm_ref_meta(_vp(vals), _vp(E), _vp(B), _vp(C_ws), M, N, K, N, N, _lib.FP16, None,
                                       _vp(ws), ws.numel() * 4, stream))
        C_na = torch.full((M, N), float("nan"), dtype=torch.float16, device=DEV)
        _lib.check(L.s24_spmm_ref_meta_noalloc(_vp(vals), _vp(E), _vp(B), _vp(C_na), M, N, K, N, N, _lib.FP16, None, stream))
        torch.cuda.synchronize()
        assert L.s24_device_status(None) == 0, _lib.last_error()
        assert torch.equal(C_na, C_ws)
        rows = slice(8064, 8192)
        ref = from_bits(ap[rows], torch.float16, DEV).float() @ B.float()
        torch.testing.assert_close(C_na[rows].float(), ref, rtol=1e-2, atol=1e-2 + 8e-3 * float(ref.abs().max()))


def test_noalloc_entry_checks_shapes_before_sizing_its_scratch():
    """dimensions whose record count would overflow, or that break the divisibility rules, are
    refused before anything touches the shared buffer"""
    from s24 import _lib
    L = _lib.lib()
    dummy = torch.empty(16, dtype=torch.float16, device=DEV)
    for M, K in ((1 << 40, 1 << 40), (100, 128), (128, 100), (0, 128)):
        rc = L.s24_spmm_ref_meta_noalloc(_vp(dummy), _vp(dummy), _vp(dummy), _vp(dummy), M, 128, K, 128, 128,
                                         _lib.FP16, None, None)
        assert rc == _lib.ERR_SHAPE, (M, K, _lib.last_error())
        rc = L.s24_spmm_ref_meta(_vp(dummy), _vp(dummy), _vp(dummy), _vp(dummy), M, 128, K, 128, 128,
                                 _lib.FP16, None, _vp(dummy), 32, None)
        assert rc == _lib.ERR_SHAPE, (M, K, _lib.last_error())


def test_noalloc_entry_rejects_problems_beyond_its_buffer():
    from s24 import _lib
    L = _lib.lib()
    M = K = 16384                      # metadata 32 MiB > the 8 MiB built-in buffer
    assert M * K // 8 > _lib.STATIC_SCRATCH_BYTES
    dummy = torch.empty(16, dtype=torch.float16, device=DEV)   # never touched: the size check comes first
    rc = L.s24_spmm_ref_meta_noalloc(_vp(dummy), _vp(dummy), _vp(dummy), _vp(dummy), M, 128, K, 128, 128,
                                     _lib.FP16, None, None)
    assert rc == _lib.ERR_SHAPE
    msg = _lib.last_error()
    assert "built-in buffer" in msg and str(M * K // 8) in msg and str(_lib.STATIC_SCRATCH_BYTES) in msg
