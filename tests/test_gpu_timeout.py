"""The bounded-wait error path of the GEMM kernels, exercised without hanging anything.

Every barrier wait in the kernels gives up after a limit; the kernel then records a code in a
status word, all roles leave their loops, tensor memory is freed and the kernel returns, so a
protocol error (or a peer that never delivers) shows up as S24_ERR_TIMEOUT from
s24_device_status instead of a hung GPU.  These tests make such a wait run out on purpose through
`s24_selftest_timeout`, whose waits are limited to one millisecond: first a bare wait on a barrier
that nothing completes, then the real GEMM kernel with its producer stopped after the first
k-block.  After each, the status word must be set once, cleared by the read, and an ordinary GEMM
on the same context must still give the right answer.
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


def _operands(M, K, N, seed):
    A = randn((M, K), torch.float16, seed)
    B = randn((K, N), torch.float16, seed + 1).to(DEV)
    ap = oracle.prune(bits(A), oracle.FP16)
    vals, ml, _ = oracle.compress(ap, oracle.FP16)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    return from_bits(vals, torch.float16, DEV), tc, B, ap


def _ordinary_gemm_is_right(L, _lib):
    M, K, N = 256, 512, 256
    v, tc, B, ap = _operands(M, K, N, 77)
    C = torch.empty(M, N, dtype=torch.float16, device=DEV)
    _lib.check(L.s24_spmm(_vp(v), _vp(tc), _vp(B), _vp(C), M, N, K, N, N, _lib.FP16, None, None))
    assert L.s24_device_status(None) == 0, _lib.last_error()
    ref = from_bits(ap, torch.float16, DEV).float() @ B.float()
    torch.testing.assert_close(C.float(), ref, rtol=1e-2, atol=1e-2 + 4e-3 * float(ref.abs().max()))


def test_a_wait_that_nothing_satisfies_runs_out_and_is_reported():
    from s24 import _lib
    L = _lib.lib()
    with torch.cuda.device(DEV):
        assert L.s24_device_status(None) == 0, _lib.last_error()
        _lib.check(L.s24_selftest_timeout(0, None, None, None, None, 0, 0, 0, _lib.FP16, None, None))
        assert L.s24_device_status(None) == _lib.ERR_TIMEOUT
        assert "code 7" in _lib.last_error()
        assert L.s24_device_status(None) == 0          # reading the word cleared it
        _ordinary_gemm_is_right(L, _lib)


@pytest.mark.parametrize("bm,bn", [(128, 128), (256, 128), (512, 224)])
def test_a_starved_gemm_unwinds_frees_tensor_memory_and_returns(bm, bn):
    """producer stops after one of two k-blocks: the MMA issuer waits for the second stage, the
    epilogue warps for an accumulator; both give up after 1 ms, the kernel returns"""
    from s24 import _lib
    L = _lib.lib()
    M, K, N = 128, 256, 128
    with torch.cuda.device(DEV):
        v, tc, B, _ = _operands(M, K, N, 5)
        C = torch.zeros(M, N, dtype=torch.float16, device=DEV)
        cfg = _lib.TileCfg(bm, bn, 0, 0)
        _lib.check(L.s24_selftest_timeout(1, _vp(v), _vp(tc), _vp(B), _vp(C), M, N, K, _lib.FP16, ctypes.byref(cfg), None))
        assert L.s24_device_status(None) == _lib.ERR_TIMEOUT
        msg = _lib.last_error()
        assert "code 2" in msg or "code 4" in msg, msg   # MMA issuer waiting for data, or epilogue waiting for the accumulator
        assert L.s24_device_status(None) == 0
        # tensor memory was handed back: the next kernels on this SM can allocate all of it again
        for _ in range(3):
            _ordinary_gemm_is_right(L, _lib)


def test_selftest_rejects_bad_requests():
    from s24 import _lib
    L = _lib.lib()
    assert L.s24_selftest_timeout(2, None, None, None, None, 0, 0, 0, _lib.FP16, None, None) == _lib.ERR_INVALID_ARG
    d = torch.empty(16, dtype=torch.float16, device=DEV)
    assert L.s24_selftest_timeout(1, _vp(d), _vp(d), _vp(d), _vp(d), 128, 128, 128, _lib.FP16, None, None) == _lib.ERR_SHAPE
