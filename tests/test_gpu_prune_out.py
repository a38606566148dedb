"""GPU parity of the fused-output-prune GEMM (the reference's v10.1) and of its separated
two-kernel comparison (v10.2).

Oracle, as the reference's own check builds it (compression/kernels/10.1_prune_acc.py:727-730):
C_ref = A_pruned @ B, then prune_2_4 and compress_dense_to_sparse of C_ref.  The low bits of an
accumulator depend on summation order (and the kernel ranks the sums after rounding them to the
output type), so the keep mask is required to match the oracle's prune of the fp32 product
except in groups whose 2nd and 3rd largest values are closer than the GEMM tolerance
(rtol = atol = 1e-2); where masks agree the stored values must agree within that tolerance, and
where they do not the stored values must still be genuine elements of the group.  Independently of
any tolerance, the fused output must equal, bit for bit, the oracle's prune (lower index on ties)
of the dense C the plain kernel stores for the same operands and tile.
"""
import numpy as np
import pytest
import torch

from util import ODT, bits, from_bits, load_dropin, oracle, randn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-2


@pytest.fixture(scope="module")
def mods():
    import s24
    torch.backends.cuda.matmul.allow_tf32 = False
    return {"s24": s24, "v101": load_dropin("kernels/10.1_prune_acc.py"),
            "v102": load_dropin("dev/10.2_prune_acc_2_kernel.py")}


def _codes_to_mask(meta_logical: np.ndarray) -> np.ndarray:
    """(M, N/16) int16 -> (M, N/4) keep masks (bit i = element i stored)"""
    w = meta_logical.view(np.uint16).astype(np.uint32)
    codes = np.stack([(w >> (4 * j)) & 0xF for j in range(4)], axis=-1).reshape(w.shape[0], -1)
    return ((1 << (codes & 3)) | (1 << (codes >> 2))).astype(np.uint8)


def _check_against_oracle(c_vals, c_meta_ref, C32, dtype):
    """c_vals (M, N/2) torch, c_meta_ref (M/16, N) int16 torch, C32 (M, N) fp32 torch on GPU"""
    M, N = C32.shape
    c32 = C32.cpu().numpy()
    want_p, want_mask = oracle.prune_f32(c32, oracle.MODE_SIGNED, oracle.TIE_LOWER, return_mask=True)
    off = oracle.meta_offsets(M, N // 16)
    got_ml = c_meta_ref.cpu().numpy().reshape(-1)[off].reshape(M, N // 16)
    got_mask = _codes_to_mask(got_ml)
    # every code is one of the six valid 2:4 codes
    assert np.isin(got_mask, [0b0011, 0b0101, 0b0110, 0b1001, 0b1010, 0b1100]).all()
    groups = c32.reshape(M, N // 4, 4)
    srt = np.sort(groups, axis=-1)
    second, third = srt[..., 2], srt[..., 1]
    near_tie = np.abs(second - third) <= TOL + TOL * np.abs(second)
    differ = got_mask != want_mask
    assert not (differ & ~near_tie).any(), f"{int((differ & ~near_tie).sum())} masks differ away from near-ties"
    # values: stored pair = the two masked elements in index order
    got_v = c_vals.float().cpu().numpy().reshape(M, N // 4, 2)
    bitsel = (got_mask[..., None] >> np.arange(4)) & 1
    idx = np.argsort(-bitsel, axis=-1, kind="stable")[..., :2]
    idx.sort(axis=-1)
    picked = np.take_along_axis(groups, idx, axis=-1)
    np.testing.assert_allclose(got_v, picked, rtol=TOL, atol=TOL + 2e-3 * float(np.abs(c32).max()))
    return float(differ.mean()), float(near_tie.mean())


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 512, 384), (384, 256, 1024), (1024, 1152, 512), (1536, 896, 256),
                                   (160, 256, 192), (32, 128, 64)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [None, {"BM": 128, "BN": 128}, {"BM": 256, "BN": 128}, {"BM": 256, "BN": 256}, {"BM": 512, "BN": 224}])
def test_fused_output_prune(mods, M, N, K, dtype, cfg):
    s24 = mods["s24"]
    A = randn((M, K), dtype, M + N + K)
    B = randn((K, N), dtype, M + N + K + 1)
    vals, _, tc = s24.prune_compress(A.to(DEV), want_ref=False, want_tc=True)
    cv, ce, ct = s24.spmm_prune_out(vals, tc, B.to(DEV), want_ref=True, want_tc=True, manual_config=cfg)
    from s24 import _lib
    assert _lib.lib().s24_device_status(None) == 0, _lib.last_error()
    assert cv.shape == (M, N // 2) and ce.shape == (M // 16, N) and ce.dtype == torch.int16
    Ap = from_bits(oracle.prune(bits(A), ODT[dtype]), dtype, DEV).float()   # pruned by the CPU oracle, not by the library
    C32 = Ap @ B.to(DEV).float()
    _check_against_oracle(cv, ce, C32, dtype)
    # the two metadata layouts describe the same array
    assert torch.equal(s24.meta_convert(ct, "tc", "ref", M, N), ce)


@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (1024, 1152, 512), (160, 256, 192)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [{"BM": 128, "BN": 128}, {"BM": 256, "BN": 128}, {"BM": 256, "BN": 256}, {"BM": 512, "BN": 224}])
def test_fused_output_is_prune_compress_of_the_plain_kernels_c(mods, M, N, K, dtype, cfg):
    """decompress(C_vals, C_meta) == oracle.prune(C) with C from s24_spmm on the same tile: no tolerance"""
    s24 = mods["s24"]
    A = randn((M, K), dtype, 7 * M + N + K)
    B = randn((K, N), dtype, 7 * M + N + K + 1)
    vals, _, tc = s24.prune_compress(A.to(DEV), want_ref=False, want_tc=True)
    C = s24.spmm(vals, tc, B.to(DEV), manual_config=cfg)
    cv, ce, ct = s24.spmm_prune_out(vals, tc, B.to(DEV), want_ref=True, want_tc=True, manual_config=cfg)
    want = oracle.prune(bits(C), ODT[dtype], oracle.MODE_SIGNED, oracle.TIE_LOWER)
    off = oracle.meta_offsets(M, N // 16)
    ml = ce.cpu().numpy().reshape(-1)[off].reshape(M, N // 16)
    got = oracle.decompress(bits(cv), ml)
    assert np.array_equal(got & 0x7FFF, want & 0x7FFF)                  # same survivors in the same places
    nz = (want & 0x7FFF) != 0
    assert np.array_equal(got[nz], want[nz])                            # with their signs
    assert np.isin(_codes_to_mask(ml), [0b0011, 0b0101, 0b0110, 0b1001, 0b1010, 0b1100]).all()
    assert torch.equal(s24.meta_convert(ct, "tc", "ref", M, N), ce)


def test_exact_case_is_bit_identical(mods):
    """small-integer operands make every accumulator exact, so no near-tie carve-out applies:
    the fused epilogue must equal compress(prune(C)) of the oracle bit for bit (lower index wins)."""
    s24 = mods["s24"]
    M, N, K = 256, 512, 256
    g = torch.Generator().manual_seed(3)
    A = torch.randint(-2, 3, (M, K), generator=g).to(torch.float16)
    B = torch.randint(-2, 3, (K, N), generator=g).to(torch.float16)
    ap = oracle.prune(bits(A), oracle.FP16)
    vals, ml, e = oracle.compress(ap, oracle.FP16)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    cv, ce, _ = s24.spmm_prune_out(from_bits(vals, torch.float16, DEV), tc, B.to(DEV))
    c32, _ = oracle.gemm_f32acc(ap, bits(B), oracle.FP16)
    want_p, want_mask = oracle.prune_f32(c32, oracle.MODE_SIGNED, oracle.TIE_LOWER, return_mask=True)
    off = oracle.meta_offsets(M, N // 16)
    got_mask = _codes_to_mask(ce.cpu().numpy().reshape(-1)[off].reshape(M, N // 16))
    assert np.array_equal(got_mask, want_mask)
    got_v = cv.float().cpu().numpy().reshape(M, N // 4, 2)
    bitsel = (want_mask[..., None] >> np.arange(4)) & 1
    idx = np.argsort(-bitsel, axis=-1, kind="stable")[..., :2]
    idx.sort(axis=-1)
    assert np.array_equal(got_v, np.take_along_axis(c32.reshape(M, N // 4, 4), idx, axis=-1))


def test_v101_dropin_entry_point_and_reference_style_check(mods):
    """run_sparse_ws_matmul(A_comp, E, B) -> (C_vals, C_meta) called like the reference's own
    self-check (10.1_prune_acc.py:715-781), including its relaxed block test."""
    s24 = mods["s24"]
    M, N, K = 1024, 2048, 1024
    A = randn((M, K), torch.float16, 21)
    B = randn((K, N), torch.float16, 22)
    ap = oracle.prune(bits(A), oracle.FP16)
    vals, ml, e = oracle.compress(ap, oracle.FP16)
    E = torch.from_numpy(e).to(DEV).view(M // 16, K)
    D_comp, D_meta = mods["v101"].run_sparse_ws_matmul(from_bits(vals, torch.float16, DEV), E, B.to(DEV))
    assert D_comp.shape == (M, N // 2) and D_meta.shape == (M // 16, N)
    C32 = from_bits(ap, torch.float16, DEV).float() @ B.to(DEV).float()
    _check_against_oracle(D_comp, D_meta, C32, torch.float16)
    # reference-style: compressed blocks that differ by > 1e-1 must consist of genuine elements
    C_ref = C32.to(torch.float16)
    cb = oracle.prune(bits(C_ref), oracle.FP16)
    cvals, _, _ = oracle.compress(cb, oracle.FP16)
    D = D_comp.float().cpu().view(-1, 2)
    Cc = from_bits(cvals, torch.float16).float().view(-1, 2)
    bad = (D - Cc).abs().max(dim=-1).values > 1e-1
    if bad.any():
        dense = C_ref.float().cpu().view(-1, 4)[bad]
        dist = (D[bad].unsqueeze(2) - dense.unsqueeze(1)).abs().min(dim=2).values
        assert float(dist.max()) <= 1e-2 + 1e-1 * float(dense.abs().max())


def test_v102_separated_path(mods):
    s24 = mods["s24"]
    M, N, K = 512, 1024, 768
    A = randn((M, K), torch.float16, 31)
    B = randn((K, N), torch.float16, 32)
    ap = oracle.prune(bits(A), oracle.FP16)
    vals, ml, e = oracle.compress(ap, oracle.FP16)
    E = torch.from_numpy(e).to(DEV).view(M // 16, K)
    C, cv, ce = mods["v102"].run_matmul_then_compress_separate(from_bits(vals, torch.float16, DEV), E, B.to(DEV))
    ref = from_bits(ap, torch.float16, DEV).float() @ B.to(DEV).float()
    torch.testing.assert_close(C.float(), ref, rtol=1e-2, atol=1e-2 + 4e-3 * float(ref.abs().max()))
    # second kernel: bit-exact prune+compress of the dense C it was given (strict >, higher index wins)
    want_p = oracle.prune(bits(C), oracle.FP16, oracle.MODE_SIGNED, oracle.TIE_HIGHER)
    want_v, _, want_e = oracle.compress(want_p, oracle.FP16)
    assert np.array_equal(bits(cv), want_v) and np.array_equal(ce.cpu().numpy(), want_e)


def test_chaining_fused_output_into_next_gemm(mods):
    """the compressed output with tensor-core-layout metadata is a valid sparse A operand"""
    s24 = mods["s24"]
    M, N, K, N2 = 256, 512, 256, 384
    A = randn((M, K), torch.float16, 41)
    B = randn((K, N), torch.float16, 42, scale=0.1)
    B2 = randn((N, N2), torch.float16, 43, scale=0.1)
    vals, _, tc = s24.prune_compress(A.to(DEV), want_ref=False, want_tc=True)
    cv, ce, ct = s24.spmm_prune_out(vals, tc, B.to(DEV), want_ref=True, want_tc=True)
    D = s24.spmm(cv, ct, B2.to(DEV))
    # decompress (cv, ce) on the CPU and multiply
    off = oracle.meta_offsets(M, N // 16)
    ml = ce.cpu().numpy().reshape(-1)[off].reshape(M, N // 16)
    dense = from_bits(oracle.decompress(bits(cv), ml), torch.float16, DEV).float()
    ref = dense @ B2.to(DEV).float()
    torch.testing.assert_close(D.float(), ref, rtol=1e-2, atol=1e-2 + 4e-3 * float(ref.abs().max()))
