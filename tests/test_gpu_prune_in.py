"""GPU parity of the fused-input-prune GEMM (the reference's v7.8.1): C = prune_2_4(A) @ B computed
from the DENSE A in one kernel.

Checks, as the reference's own (compression/kernels/7.8.1_prune_ws.py:712-716: C against
prune_2_4(A) @ B): the result is within rtol = atol = 1e-2 of an fp32-accumulated product of the
oracle-pruned A; with B = I (and the reference's tie rule) it is the oracle-pruned matrix itself;
and it is bit-identical to the two-kernel path (prune+compress, then the sparse GEMM; a dot product runs over K in the same
order whatever the MMA's N), which pins the in-kernel values, metadata records and their shared-memory layout.
"""
import numpy as np
import pytest
import torch

from util import ODT, MODE, TIE, bits, from_bits, load_dropin, oracle, randn, tie_heavy

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL = ATOL = 1e-2


@pytest.fixture(scope="module")
def mods():
    import s24
    torch.backends.cuda.matmul.allow_tf32 = False
    return {"s24": s24, "v781": load_dropin("kernels/7.8.1_prune_ws.py")}


def _status_ok():
    from s24 import _lib
    rc = _lib.lib().s24_device_status(None)
    assert rc == 0, _lib.last_error()


def _reference(A, B, dtype, mode="signed", tie="reference"):
    ap = oracle.prune(bits(A), ODT[dtype], MODE[mode], TIE[tie])
    return from_bits(ap, dtype, DEV).float() @ B.to(DEV).float(), ap


def _check(C, ref32):
    torch.testing.assert_close(C.float(), ref32.to(C.dtype).float(), rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(C.float(), ref32, rtol=RTOL, atol=ATOL + 4e-3 * float(ref32.abs().max()))


def test_identity_b_reveals_pruned_a(mods):
    s24 = mods["s24"]
    M = K = 512
    A = randn((M, K), torch.float16, 71)
    # with the reference's tie rule the survivors sit where the oracle's (torch.topk) do
    C = s24.spmm_prune_in(A.to(DEV), torch.eye(K, dtype=torch.float16, device=DEV), tie="reference")
    _status_ok()
    ap = oracle.prune(bits(A), oracle.FP16)
    assert torch.equal(C.float().cpu(), from_bits(ap, torch.float16).float())


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 8, 128), (256, 24, 256), (256, 256, 512), (384, 200, 384),
                                   (512, 1032, 1280), (1024, 768, 2048), (256, 256, 16384), (4096, 128, 256),
                                   (2048, 8192, 2048), (256, 480, 256), (256, 488, 384), (512, 728, 256), (256, 968, 128),
                                   (32, 8, 64), (160, 72, 192), (416, 496, 320)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prune_in_vs_fp32_reference_and_two_kernel_path(mods, M, N, K, dtype):
    s24 = mods["s24"]
    A = randn((M, K), dtype, 700 + M + N + K)
    B = randn((K, N), dtype, 701 + M + N + K)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = mods["v781"].run_sparse_ws_matmul(Ad, Bd)
    _status_ok()
    assert C.shape == (M, N) and C.dtype == dtype
    ref32, _ = _reference(A, B, dtype, tie="higher")   # the shim's default: the reference kernel's strict compare
    _check(C, ref32)
    # and under the torch function's tie rule against the oracle's default
    ref32, _ = _reference(A, B, dtype)
    _check(s24.spmm_prune_in(Ad, Bd, tie="reference"), ref32)
    vals, _, tc = s24.prune_compress(Ad, tie="higher", want_ref=False, want_tc=True)
    C2 = s24.spmm(vals, tc, Bd, manual_config={"BM": 512, "BN": 224})
    assert torch.equal(C.view(torch.int16), C2.view(torch.int16))


@pytest.mark.parametrize("mode", ["signed", "magnitude"])
@pytest.mark.parametrize("tie", ["reference", "lower", "higher"])
def test_modes_and_tie_rules_on_tie_heavy_input(mods, mode, tie):
    """A tie decides which of two equal values survives, i.e. which row of B it multiplies, so C
    depends on the rule: each rule is checked against the oracle run with the same rule, and
    bit for bit against the two-kernel path."""
    s24 = mods["s24"]
    M, N, K = 384, 136, 640
    A = tie_heavy((M, K), torch.float16, 73)
    B = randn((K, N), torch.float16, 74)
    Ad, Bd = A.to(DEV), B.to(DEV)
    C = s24.spmm_prune_in(Ad, Bd, mode=mode, tie=tie)
    _status_ok()
    ref32, _ = _reference(A, B, torch.float16, mode, tie)
    _check(C, ref32)
    vals, _, tc = s24.prune_compress(Ad, mode=mode, tie=tie, want_ref=False, want_tc=True)
    C2 = s24.spmm(vals, tc, Bd, manual_config={"BM": 512, "BN": 224})
    assert torch.equal(C.view(torch.int16), C2.view(torch.int16))


def test_strided_and_narrowly_aligned_operands(mods):
    """A with a row stride larger than K and a base that is only 16-byte aligned (the kernel
    falls back to 16-byte loads), B and C as column slices of wider tensors."""
    s24 = mods["s24"]
    M, N, K = 256, 320, 512
    A = randn((M, K), torch.float16, 75)
    B = randn((K, N), torch.float16, 76)
    wideA = torch.zeros((M, K + 24), dtype=torch.float16, device=DEV)
    Av = wideA[:, 8:8 + K]
    Av.copy_(A)
    assert Av.data_ptr() % 32 == 16
    wideB = torch.zeros((K, N + 64), dtype=torch.float16, device=DEV)
    Bv = wideB[:, 32:32 + N]
    Bv.copy_(B)
    wideC = torch.full((M, N + 16), 7.0, dtype=torch.float16, device=DEV)
    Cv = wideC[:, 8:8 + N]
    out = s24.spmm_prune_in(Av, Bv, tie="reference", out=Cv)
    _status_ok()
    assert out.data_ptr() == Cv.data_ptr()
    ref32, _ = _reference(A, B, torch.float16)
    _check(Cv, ref32)
    assert bool((wideC[:, :8] == 7.0).all()) and bool((wideC[:, 8 + N:] == 7.0).all())


def test_rejects_bad_arguments(mods):
    s24 = mods["s24"]
    A = torch.zeros((128, 128), dtype=torch.float16, device=DEV)
    B = torch.zeros((128, 64), dtype=torch.float16, device=DEV)
    with pytest.raises(RuntimeError):
        s24.spmm_prune_in(A[:48], B)                      # M % 32
    with pytest.raises(RuntimeError):
        s24.spmm_prune_in(A, B[:, :12])                   # N % 8
    with pytest.raises(RuntimeError):
        s24.spmm_prune_in(A, B.to(torch.bfloat16))        # dtype mismatch
    with pytest.raises(RuntimeError):
        s24.spmm_prune_in(A, B, out=torch.empty((128, 32), dtype=torch.float16, device=DEV))
    from s24 import _lib
    rc = _lib.lib().s24_spmm_prune_in(None, 128, B.data_ptr(), A.data_ptr(), 128, 64, 128, 64, 64, 0, 0, 0, None)
    assert rc != 0 and "null" in _lib.last_error()
    rc = _lib.lib().s24_spmm_prune_in(A.data_ptr(), 64, B.data_ptr(), A.data_ptr(), 128, 64, 128, 64, 64, 0, 0, 0, None)
    assert rc != 0 and "lda" in _lib.last_error()
