"""GPU parity of prune / compress / fused prune+compress against the oracle and the golden
vectors, through the drop-in modules and the C ABI.  Everything is bit-exact."""
import zlib

import numpy as np
import pytest
import torch

from util import ODT, MODE, TIE, bits, from_bits, load_dropin, oracle, randn, tie_heavy

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def mods():
    import s24
    return {"s24": s24, "prune": load_dropin("prune.py"), "compress": load_dropin("compress_2_4.py"),
            "two": load_dropin("kernels/11.1_2_kernel_baseline.py")}


GOLD = [("randn_f16", torch.float16), ("randn_bf16", torch.bfloat16), ("ties_f16", torch.float16),
        ("ties_bf16", torch.bfloat16), ("special_f16", torch.float16)]


@pytest.mark.parametrize("name,dtype", GOLD)
def test_golden_vectors_through_dropin_api(mods, golden, name, dtype):
    A = from_bits(golden[f"{name}.A"], dtype, DEV)
    M, K = A.shape
    pruned = mods["prune"].prune_2_4(A)
    assert np.array_equal(bits(pruned), golden[f"{name}.pruned"])
    vals, meta = mods["compress"].compress_dense_to_sparse(pruned)
    assert tuple(meta.shape) == (M // 2, K // 8) and meta.dtype == torch.int16
    assert np.array_equal(bits(vals), golden[f"{name}.vals"])
    assert np.array_equal(meta.view(M // 16, K).cpu().numpy(), golden[f"{name}.E"])
    # magnitude mode
    pm = mods["prune"].prune_2_4(A, mode="magnitude")
    assert np.array_equal(bits(pm), golden[f"{name}.pruned_mag"])
    # fused kernel == prune followed by compress
    v2, e2, _ = mods["s24"].prune_compress(A, mode="signed", tie="reference")
    assert np.array_equal(bits(v2), golden[f"{name}.vals"])
    assert np.array_equal(e2.cpu().numpy(), golden[f"{name}.E"])
    v3, e3, _ = mods["s24"].prune_compress(A, mode="magnitude", tie="reference")
    assert np.array_equal(bits(v3), golden[f"{name}.vals_mag"])
    assert np.array_equal(e3.cpu().numpy(), golden[f"{name}.E_mag"])


def test_encoder_table_on_unpruned_input(mods, golden):
    d = from_bits(golden["flags_f16.dense"], torch.float16, DEV)
    vals, meta = mods["compress"].compress_dense_to_sparse(d)
    assert np.array_equal(bits(vals), golden["flags_f16.vals"])
    assert np.array_equal(meta.view(4, 128).cpu().numpy(), golden["flags_f16.E"])


def test_meta_offsets_helper(mods, golden):
    for m, nc in ((32, 4), (64, 8), (128, 16)):
        off = mods["compress"]._calculate_meta_reordering_offsets(m, nc, "cpu")
        assert np.array_equal(off.numpy(), golden[f"offsets_{m}_{nc}"])


SHAPES = [(32, 64), (32, 192), (64, 128), (96, 320), (128, 128), (160, 448), (256, 1152), (2048, 2048)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode,tie", [("signed", "reference"), ("signed", "lower"), ("signed", "higher"),
                                      ("magnitude", "reference"), ("magnitude", "lower")])
def test_fused_kernel_vs_oracle(mods, shape, dtype, mode, tie):
    seed = zlib.crc32(repr((shape, str(dtype), mode, tie)).encode()) % 10000
    gen = tie_heavy if shape[0] <= 96 else randn
    A = gen(shape, dtype, seed)
    if dtype == torch.bfloat16 and gen is randn:
        A = (A.float() * 0.02).to(dtype)
    ab = bits(A)
    want_p = oracle.prune(ab, ODT[dtype], MODE[mode], TIE[tie])
    want_v, want_ml, want_e = oracle.compress(want_p, ODT[dtype])
    M, K = shape
    # the tensor-core layout comes in whole (128-row, 128-column) records: shapes that cover the last
    # ones partly are included, the words outside the matrix hold the filler code
    v, e, tc = mods["s24"].prune_compress(A.to(DEV), mode=mode, tie=tie, want_ref=True, want_tc=True)
    assert np.array_equal(bits(v), want_v)
    assert np.array_equal(e.cpu().numpy(), want_e)
    assert np.array_equal(tc.cpu().numpy().view(np.uint32), oracle.meta_tc(want_ml, K))
    # dense prune
    p = mods["s24"].prune(A.to(DEV), mode=mode, tie=tie)
    assert np.array_equal(bits(p), want_p)
    # compress of the pruned matrix gives the same pair
    v2, e2, _ = mods["s24"].compress(p)
    assert np.array_equal(bits(v2), want_v) and np.array_equal(e2.cpu().numpy(), want_e)


def test_prune_accepts_any_leading_shape_and_odd_group_counts(mods):
    for shape in [(3, 5, 12), (7, 4), (1, 20), (2, 3, 4, 8)]:
        A = tie_heavy(shape, torch.float16, 7)
        got = mods["prune"].prune_2_4(A.to(DEV))
        assert got.shape == A.shape
        want = oracle.prune(bits(A).reshape(-1, shape[-1]), oracle.FP16)
        assert np.array_equal(bits(got).reshape(-1, shape[-1]), want)
    # a view with an offset of 4 elements: 8-byte aligned only
    base = tie_heavy((1, 36), torch.float16, 9).to(DEV)
    got = mods["prune"].prune_2_4(base[:, 4:])
    assert np.array_equal(bits(got), oracle.prune(bits(base[:, 4:]), oracle.FP16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prune_in_place_through_the_c_abi(mods, dtype):
    """s24_prune documents that `out` may equal `A`: prune a buffer onto itself, 16-byte aligned and
    (a view 4 elements in) 8-byte aligned only, large enough for the grid-stride loop to wrap"""
    import ctypes
    from s24 import _lib
    L = _lib.lib()
    for offset, n in ((0, 1 << 22), (4, (1 << 22) - 8), (0, 2048)):
        buf = tie_heavy((1, (1 << 22) + 8), dtype, 31 + offset).to(DEV) if n < 4096 else randn((1, (1 << 22) + 8), dtype, 33 + offset).to(DEV)
        view = buf[0, offset:offset + n]
        want = oracle.prune(bits(view).reshape(-1, 4), ODT[dtype]).reshape(-1)
        ptr = ctypes.c_void_p(view.data_ptr())
        _lib.check(L.s24_prune(ptr, ptr, n, _lib.FP16 if dtype == torch.float16 else _lib.BF16, _lib.MODE_SIGNED,
                               _lib.TIE_REFERENCE, None))
        torch.cuda.synchronize()
        assert np.array_equal(bits(view), want)


def test_input_is_not_modified_and_strided_rows_work(mods):
    big = randn((64, 256), torch.float16, 3).to(DEV)
    A = big[:, :128]                      # row stride 256, not contiguous
    keep = A.clone()
    v, e, _ = mods["s24"].prune_compress(A)
    assert torch.equal(A, keep)
    want_v, _, want_e = oracle.compress(oracle.prune(bits(keep), oracle.FP16), oracle.FP16)
    assert np.array_equal(bits(v), want_v) and np.array_equal(e.cpu().numpy(), want_e)


@pytest.mark.parametrize("name,dtype", [("int8", torch.int8), ("int32", torch.int32), ("float32", torch.float32)])
def test_other_element_types_of_compress(mods, name, dtype):
    """compress_dense_to_sparse for int8 / int32 / float32 (compress_2_4.py:41-47,73-76,144-154) through the
    drop-in: the reference's golden outputs, then larger random patterns and a strided view against the oracle"""
    from pathlib import Path
    c = mods["compress"].compress_dense_to_sparse
    g = dict(np.load(Path(__file__).resolve().parent / "golden" / "golden_other_dtypes.npz"))
    v, m = c(torch.from_numpy(g[f"{name}.dense"]).to(DEV))
    assert v.dtype == dtype and tuple(m.shape) == g[f"{name}.meta"].shape
    assert np.array_equal(v.cpu().numpy().view(np.uint8), g[f"{name}.vals"].view(np.uint8))
    assert np.array_equal(m.cpu().numpy(), g[f"{name}.meta"])
    rng = np.random.default_rng(7)
    for (M, K) in ((512, 1024), (96 if dtype != torch.int8 else 80, 2176)):
        flags = rng.integers(0, 2, size=(M, K))
        dense = (flags * rng.integers(-50, 50, size=(M, K))).astype(g[f"{name}.dense"].dtype)
        want_v, want_m = oracle.compress_other(dense)
        wide = torch.zeros(M, K + 64, dtype=dtype, device=DEV)
        wide[:, 32:32 + K] = torch.from_numpy(dense).to(DEV)
        for src in (torch.from_numpy(dense).to(DEV), wide[:, 32:32 + K]):         # contiguous, then row stride > K
            v, m = c(src)
            assert np.array_equal(v.cpu().numpy().view(np.uint8), want_v.view(np.uint8))
            assert np.array_equal(m.cpu().numpy(), want_m)
    with pytest.raises(RuntimeError, match="divisible by"):
        c(torch.zeros(24, 128, dtype=dtype, device=DEV))
    with pytest.raises(AssertionError):
        c(torch.zeros(32, 32 if dtype == torch.int8 else 16, dtype=dtype, device=DEV))
    d = torch.zeros(0, 128, dtype=dtype, device=DEV)
    v, m = c(d)
    assert v.shape == d.shape and m.numel() == 0 and m.dtype == (torch.int32 if dtype == torch.int8 else torch.int16)


def test_error_behaviour_matches_reference(mods):
    c = mods["compress"].compress_dense_to_sparse
    with pytest.raises(ValueError):
        mods["prune"].prune_2_4(torch.zeros(4, 6, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError, match="2-dimensional"):
        c(torch.zeros(2, 32, 64, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError, match="divisible by 32"):
        c(torch.zeros(16, 64, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError, match="divisible by 16"):
        c(torch.zeros(32, 40, dtype=torch.float16, device=DEV))
    with pytest.raises(AssertionError):
        c(torch.zeros(32, 48, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError, match="Invalid datatype"):
        c(torch.zeros(32, 64, dtype=torch.float64, device=DEV))
    with pytest.raises(RuntimeError, match="Invalid datatype"):
        c(torch.zeros(32, 64, dtype=torch.int64, device=DEV))
    # empty input: returned as is with zero metadata (compress_2_4.py:67)
    d = torch.zeros(0, 64, dtype=torch.float16, device=DEV)
    v, m = c(d)
    assert v.shape == d.shape and m.numel() == 0


@pytest.mark.parametrize("M,K", [(128, 128), (256, 384), (384, 640), (1024, 2048), (2176, 1152), (32, 64), (160, 192),
                                 (416, 320), (96, 1024)])
def test_meta_layout_round_trips(mods, M, K):
    s24 = mods["s24"]
    rng = np.random.default_rng(M + K)
    codes = np.array([4, 8, 9, 12, 13, 14], dtype=np.uint16)
    nib = codes[rng.integers(0, 6, size=(M, K // 16, 4))]
    ml = (nib[..., 0] | (nib[..., 1] << 4) | (nib[..., 2] << 8) | (nib[..., 3] << 12)).astype(np.uint16).view(np.int16)
    logical = torch.from_numpy(ml).to(DEV)
    ref = s24.meta_convert(logical, "logical", "ref", M, K)
    off = oracle.meta_offsets(M, K // 16)
    want_ref = np.empty(M * K // 16, np.int16)
    want_ref[off] = ml.reshape(-1)
    assert np.array_equal(ref.cpu().numpy().reshape(-1), want_ref)
    tc = s24.meta_convert(ref, "ref", "tc", M, K)
    assert np.array_equal(tc.cpu().numpy().view(np.uint32), oracle.meta_tc(ml, K))
    back = s24.meta_convert(tc, "tc", "logical", M, K)
    assert np.array_equal(back.cpu().numpy(), ml)
    ref2 = s24.meta_convert(tc, "tc", "ref", M, K)
    assert torch.equal(ref2, ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_full_size_properties(mods, dtype):
    """16384 x 16384 (the bandwidth configuration): too big for the CPU oracle end to end,
    so check size-independent properties on the GPU plus sampled row panels on the CPU."""
    s24 = mods["s24"]
    M = K = 16384
    g = torch.Generator(device=DEV).manual_seed(2014)
    A = torch.randn(M, K, generator=g, device=DEV, dtype=torch.float32).to(dtype)
    if dtype == torch.bfloat16:
        A = (A.float() * 0.02).to(dtype)
    v, e, tc = s24.prune_compress(A, want_ref=True, want_tc=True)
    p = s24.prune(A)
    # (1) exactly two survivors per group, survivors untouched
    nz = (p.view(torch.int16) & 0x7FFF) != 0
    assert int(nz.view(M, K // 4, 4).sum(-1).max()) <= 2
    assert torch.equal(torch.where(nz, p, torch.zeros_like(p)), torch.where(nz, A, torch.zeros_like(A)))
    # (2) decompressing (values, metadata) gives back the dense pruned matrix
    logical = s24.meta_convert(e, "ref", "logical", M, K)
    codes = torch.stack([(logical.view(M, K // 16, 1).to(torch.int32) >> (4 * j)) & 0xF for j in range(4)], -1).view(M, K // 4)
    idx0, idx1 = (codes & 3).long(), (codes >> 2).long()
    dense = torch.zeros(M, K // 4, 4, dtype=dtype, device=DEV)
    vv = v.view(M, K // 4, 2)
    dense.scatter_(2, idx1.unsqueeze(-1), vv[..., 1:2])
    dense.scatter_(2, idx0.unsqueeze(-1), vv[..., 0:1])
    assert torch.equal(dense.view(M, K).view(torch.int16) & 0x7FFF, p.view(torch.int16) & 0x7FFF)
    # (3) both metadata layouts describe the same logical array
    assert torch.equal(s24.meta_convert(tc, "tc", "ref", M, K), e)
    # (4) sampled panels against the CPU oracle, bit for bit
    for r0 in (0, 8192 - 64, M - 128):
        ab = bits(A[r0:r0 + 128])
        want_p = oracle.prune(ab, ODT[dtype])
        want_v, _, want_e = oracle.compress(want_p, ODT[dtype])
        assert np.array_equal(bits(p[r0:r0 + 128]), want_p)
        assert np.array_equal(bits(v[r0:r0 + 128]), want_v)
        assert np.array_equal(e[r0 // 16:r0 // 16 + 8].cpu().numpy(), want_e)


def test_index_arithmetic_beyond_2_31_elements(mods):
    """49152 x 49152 has 2.4e9 elements: element offsets no longer fit 32 bits.  Check the last
    row panels (whose offsets are the largest) against the CPU oracle, bit for bit."""
    s24 = mods["s24"]
    M = K = 49152
    A = torch.empty(M, K, dtype=torch.float16, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(49152)
    for r0 in range(0, M, 8192):          # generate in slabs to bound the fp32 temporary
        A[r0:r0 + 8192] = torch.randn(8192, K, generator=g, device=DEV, dtype=torch.float32).to(torch.float16)
    v, e, tc = s24.prune_compress(A, want_ref=True, want_tc=True)
    for r0 in (0, 43776, M - 128):        # 43776 * 49152 > 2^31
        ab = bits(A[r0:r0 + 128])
        want_p = oracle.prune(ab, oracle.FP16)
        want_v, want_ml, want_e = oracle.compress(want_p, oracle.FP16)
        assert np.array_equal(bits(v[r0:r0 + 128]), want_v)
        assert np.array_equal(e[r0 // 16:r0 // 16 + 8].cpu().numpy(), want_e)
        rec = (K // 128) * 512
        got_tc = tc[(r0 // 128) * rec:(r0 // 128 + 1) * rec].cpu().numpy().view(np.uint32)
        assert np.array_equal(got_tc, oracle.meta_tc(want_ml, K))
    del v, e, tc
    p = s24.prune(A[M - 4096:])
    assert np.array_equal(bits(p[-128:]), oracle.prune(bits(A[M - 128:]), oracle.FP16))


def test_sixteen_byte_aligned_views_take_the_narrow_access_path(mods):
    """A and the values buffer only 16-byte aligned (a view 8 elements into a row): the kernel must
    fall back from 256-bit to 128-bit accesses and still be bit-exact"""
    import ctypes
    from s24 import _lib
    M, K = 64, 256
    big = randn((M, K + 16), torch.float16, 17).to(DEV)
    A = big[:, 8:8 + K]                                   # 16-byte aligned start, row stride K + 16
    vals_store = torch.empty(M * (K // 2) + 8, dtype=torch.float16, device=DEV)
    vals = vals_store[8:]                                 # 16-byte aligned, not 32
    assert A.data_ptr() % 32 == 16 and vals.data_ptr() % 32 == 16
    e = torch.empty(M // 16, K, dtype=torch.int16, device=DEV)
    rc = _lib.lib().s24_prune_compress(ctypes.c_void_p(A.data_ptr()), M, K, K + 16, _lib.FP16, _lib.MODE_SIGNED,
                                       _lib.TIE_REFERENCE, ctypes.c_void_p(vals.data_ptr()), ctypes.c_void_p(e.data_ptr()),
                                       None, None)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    want_v, _, want_e = oracle.compress(oracle.prune(bits(A), oracle.FP16), oracle.FP16)
    assert np.array_equal(bits(vals.view(M, K // 2)), want_v) and np.array_equal(e.cpu().numpy(), want_e)


def test_relayout_of_gathered_column_shards(mods):
    s24 = mods["s24"]
    G, rows, nl = 4, 96, 72
    stage = torch.randn(G, rows, nl, device=DEV).to(torch.bfloat16)
    wide = torch.zeros(rows, G * nl + 8, dtype=torch.bfloat16, device=DEV)
    out = wide[:, :G * nl]                                   # row stride larger than the logical width
    s24.relayout_shards(stage, out)
    assert torch.equal(out, stage.permute(1, 0, 2).reshape(rows, G * nl))
    assert float(wide[:, G * nl:].abs().max()) == 0


def test_property_random_shapes_bit_exact(mods):
    """hypothesis-driven: random (M % 32 == 0, K % 64 == 0) shapes, dtypes, modes, tie rules and
    value distributions (plain randn, heavy ties, tiny magnitudes with denormals); values and both
    metadata layouts must equal the oracle's bit for bit"""
    from hypothesis import given, settings, strategies as st, HealthCheck
    s24 = mods["s24"]

    @settings(max_examples=40, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
    @given(m=st.integers(1, 16), k=st.integers(1, 12), seed=st.integers(0, 2 ** 20),
           dtype=st.sampled_from([torch.float16, torch.bfloat16]), mode=st.sampled_from(["signed", "magnitude"]),
           tie=st.sampled_from(["reference", "lower", "higher"]), kind=st.sampled_from(["randn", "ties", "tiny"]))
    def run(m, k, seed, dtype, mode, tie, kind):
        M, K = 32 * m, 64 * k
        if kind == "randn":
            A = randn((M, K), dtype, seed)
        elif kind == "ties":
            A = tie_heavy((M, K), dtype, seed)
        else:
            A = randn((M, K), dtype, seed, scale=3e-7 if dtype == torch.float16 else 1e-39)
        want_p = oracle.prune(bits(A), ODT[dtype], MODE[mode], TIE[tie])
        want_v, want_ml, want_e = oracle.compress(want_p, ODT[dtype])
        v, e, tc = s24.prune_compress(A.to(DEV), mode=mode, tie=tie, want_ref=True, want_tc=True)
        assert np.array_equal(bits(v), want_v)
        assert np.array_equal(e.cpu().numpy(), want_e)
        assert np.array_equal(tc.cpu().numpy().view(np.uint32), oracle.meta_tc(want_ml, K))
        assert np.array_equal(bits(s24.prune(A.to(DEV), mode=mode, tie=tie)), want_p)

    run()
