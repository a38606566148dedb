"""GPU parity of the tcgen05 sparse GEMM: C = prune_2_4(A) @ B against an fp32-accumulated
reference (compression/gluon_ws_sparse.py:660), rtol = atol = 1e-2, through the drop-in
launchers and the C ABI.  Small cases use the CPU oracle's GEMM; larger ones an fp32
torch matmul (TF32 off) of the oracle-pruned A."""
import numpy as np
import pytest
import torch

from util import ODT, bits, from_bits, load_dropin, oracle, randn

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL = ATOL = 1e-2


@pytest.fixture(scope="module")
def mods():
    import s24
    torch.backends.cuda.matmul.allow_tf32 = False
    return {"s24": s24, "ws": load_dropin("gluon_ws_sparse.py"), "two": load_dropin("kernels/11.1_2_kernel_baseline.py")}


def _status_ok(s24):
    from s24 import _lib
    rc = _lib.lib().s24_device_status(None)
    assert rc == 0, _lib.last_error()


def _prepare(M, K, N, dtype, seed, scale=1.0):
    A = randn((M, K), dtype, seed, scale)
    B = randn((K, N), dtype, seed + 1)
    ap = oracle.prune(bits(A), ODT[dtype])
    vals, ml, e = oracle.compress(ap, ODT[dtype])
    return A, B, ap, vals, ml, e


def _reference(ap_bits, B, dtype):
    Ap = from_bits(ap_bits, dtype, DEV).float()
    return Ap @ B.to(DEV).float()


def _check(C, ref32):
    torch.testing.assert_close(C.float(), ref32.to(C.dtype).float(), rtol=RTOL, atol=ATOL)
    # and against the unrounded sums with a little room for the output rounding
    torch.testing.assert_close(C.float(), ref32, rtol=RTOL, atol=ATOL + 4e-3 * float(ref32.abs().max()))


@pytest.mark.parametrize("cfg", [{"BM": 128, "BN": 128}, {"BM": 256, "BN": 128}, {"BM": 256, "BN": 256}, {"BM": 512, "BN": 224}])
def test_identity_b_reveals_decompressed_a(mods, cfg):
    """B = I makes C the dense 2:4 matrix itself, exactly: checks values, metadata layout
    and operand descriptors independently of any accumulation."""
    s24 = mods["s24"]
    M, K = 256, 256
    A, _, ap, vals, ml, e = _prepare(M, K, K, torch.float16, 11)
    B = torch.eye(K, dtype=torch.float16)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    C = s24.spmm(from_bits(vals, torch.float16, DEV), tc, B.to(DEV), manual_config=cfg)
    _status_ok(s24)
    assert torch.equal(C.float().cpu(), from_bits(ap, torch.float16).float())   # -0.0 == +0.0


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 8, 128), (256, 24, 256), (256, 256, 512), (384, 200, 384), (512, 1032, 1280), (1024, 768, 2048), (256, 256, 16384), (4096, 128, 256),
                                   # every shape compress_dense_to_sparse accepts (M % 32, K % 64): partly covered tiles and k-blocks
                                   (32, 8, 64), (160, 72, 192), (96, 200, 64), (416, 256, 320), (544, 232, 1088)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [None, {"BM": 128, "BN": 128}, {"BM": 256, "BN": 128}, {"BM": 256, "BN": 256}, {"BM": 512, "BN": 224}])
def test_spmm_vs_fp32_reference(mods, M, N, K, dtype, cfg):
    s24 = mods["s24"]
    A, B, ap, vals, ml, e = _prepare(M, K, N, dtype, 100 + M + N + K)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    C = s24.spmm(from_bits(vals, dtype, DEV), tc, B.to(DEV), manual_config=cfg)
    _status_ok(s24)
    assert C.shape == (M, N) and C.dtype == dtype
    _check(C, _reference(ap, B, dtype))


def test_small_case_against_cpu_oracle_gemm(mods, golden):
    s24 = mods["s24"]
    ap = oracle.prune(golden["gemm_f16.A"], oracle.FP16)
    vals, ml, e = oracle.compress(ap, oracle.FP16)
    E = torch.from_numpy(e).to(DEV)
    B = from_bits(golden["gemm_f16.B"], torch.float16, DEV)
    C = mods["ws"].run_sparse_ws_matmul(from_bits(vals, torch.float16, DEV), E, B)
    _status_ok(s24)
    want32 = torch.from_numpy(golden["gemm_f16.C_f32"]).to(DEV)
    _check(C, want32)
    c32, _ = oracle.gemm_f32acc(ap, golden["gemm_f16.B"], oracle.FP16)
    _check(C, torch.from_numpy(c32).to(DEV))


def test_dropin_launcher_with_reference_layout_metadata(mods):
    """config 1 of the benchmark: A 2048 x 2048, B 2048 x 8192, through
    run_sparse_ws_matmul(A_vals, E, B) exactly as the reference's self-check calls it."""
    s24 = mods["s24"]
    M, K, N = 2048, 2048, 8192
    A, B, ap, vals, ml, e = _prepare(M, K, N, torch.float16, 1234)
    Av = from_bits(vals, torch.float16, DEV)
    E = torch.from_numpy(e).to(DEV).view(M // 16, K)
    C = mods["ws"].run_sparse_ws_matmul(Av, E, B.to(DEV))
    _status_ok(s24)
    _check(C, _reference(ap, B, torch.float16))
    C2 = mods["ws"].run_sparse_ws_matmul(Av, E, B.to(DEV), tune=False,
                                         manual_config={"BM": 128, "BN": 128, "BK": 64, "warps": 8, "buffers": 4, "SF": 4})
    _check(C2, _reference(ap, B, torch.float16))


def test_two_kernel_entry_point(mods):
    """v11.1: dense A -> prune+compress kernel -> sparse GEMM; the metadata stays in the
    tensor-core layout between the two launches."""
    s24 = mods["s24"]
    M, K, N = 1024, 1536, 2048
    A = randn((M, K), torch.float16, 77)
    B = randn((K, N), torch.float16, 78)
    C = mods["two"].run_2_kernel_ws_matmul(A.to(DEV), B.to(DEV))
    _status_ok(s24)
    ap = oracle.prune(bits(A), oracle.FP16, oracle.MODE_SIGNED, oracle.TIE_HIGHER)
    _check(C, _reference(ap, B, torch.float16))


def test_bf16_weight_times_activation_shape(mods):
    s24 = mods["s24"]
    M, K, N = 1792, 1024, 4096      # a 1/16-scale slice of the MLP-shaped configuration
    A = randn((M, K), torch.bfloat16, 5000, scale=0.02)
    B = randn((K, N), torch.bfloat16, 5001)
    vals, _, tc = s24.prune_compress(A.to(DEV), want_ref=False, want_tc=True)
    C = s24.spmm(vals, tc, B.to(DEV))
    _status_ok(s24)
    ap = oracle.prune(bits(A), oracle.BF16)
    ref = _reference(ap, B, torch.bfloat16)
    torch.testing.assert_close(C.float(), ref, rtol=RTOL, atol=ATOL)


def test_linearity_at_full_size(mods):
    """8192^3 is too large for a CPU check: use C(B1 + B2) = C(B1) + C(B2) with small-integer
    B (exact in fp16 and in the fp32 accumulator) and compare sampled rows with torch."""
    s24 = mods["s24"]
    M = N = K = 8192
    g = torch.Generator(device=DEV).manual_seed(8192)
    A = torch.randint(-3, 4, (M, K), generator=g, device=DEV).to(torch.float16)
    B1 = torch.randint(-2, 3, (K, N), generator=g, device=DEV).to(torch.float16)
    B2 = torch.randint(-2, 3, (K, N), generator=g, device=DEV).to(torch.float16)
    vals, _, tc = s24.prune_compress(A, want_ref=False, want_tc=True)
    C1 = s24.spmm(vals, tc, B1)
    C2 = s24.spmm(vals, tc, B2)
    C12 = s24.spmm(vals, tc, B1 + B2)
    _status_ok(s24)
    # integer sums of magnitude < 2048 * ... stay exactly representable only up to 2048 in fp16;
    # compare in fp32 with one fp16 ulp of slack at the observed magnitude
    tol = float(C12.float().abs().max()) * 2 ** -10
    assert float((C12.float() - (C1.float() + C2.float())).abs().max()) <= 2 * tol + 1e-3
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8191], device=DEV)
    Ap_rows = from_bits(oracle.prune(bits(A[rows]), oracle.FP16), torch.float16, DEV)   # pruned by the CPU oracle
    ref = Ap_rows.float() @ B1.float()
    torch.testing.assert_close(C1[rows].float(), ref.to(torch.float16).float(), rtol=RTOL, atol=ATOL)


def test_strided_b_and_strided_output_through_the_c_abi(mods):
    """row strides larger than the logical widths: B a column slice of a wider matrix, C written
    into a column slice of a wider buffer (ldb, ldc > N), as the multi-GPU wrapper could do"""
    import ctypes
    from s24 import _lib
    s24 = mods["s24"]
    M, K, N = 256, 512, 328                       # N % 8 == 0 but not a multiple of 16
    A, _, ap, vals, ml, e = _prepare(M, K, 1024, torch.float16, 555)
    Bwide = randn((K, 1024), torch.float16, 556).to(DEV)
    Bv = Bwide[:, 64:64 + N]                      # ldb = 1024, 16-byte aligned start
    Cwide = torch.zeros(M, 640, dtype=torch.float16, device=DEV)
    Cv = Cwide[:, 32:32 + N]                      # ldc = 640
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    v = from_bits(vals, torch.float16, DEV)
    for cfg in (None, _lib.TileCfg(512, 224, 0, 0), _lib.TileCfg(128, 128, 0, 0)):
        Cwide.zero_()
        rc = _lib.lib().s24_spmm(ctypes.c_void_p(v.data_ptr()), ctypes.c_void_p(tc.data_ptr()),
                                 ctypes.c_void_p(Bv.data_ptr()), ctypes.c_void_p(Cv.data_ptr()), M, N, K, 1024, 640,
                                 _lib.FP16, ctypes.byref(cfg) if cfg is not None else None, None)
        assert rc == 0, _lib.last_error()
        _status_ok(s24)
        ref = from_bits(ap, torch.float16, DEV).float() @ Bv.float()
        _check(Cv, ref)
        assert float(Cwide[:, :32].abs().max()) == 0 and float(Cwide[:, 32 + N:].abs().max()) == 0   # nothing outside the slice


def test_launchers_can_be_captured_in_a_cuda_graph(mods):
    """the reference's benchmarks run every launcher under CUDA-graph capture
    (triton do_bench_cudagraph, dev/8.11_benchmark_2_kernel.py:52-61): capture the two-kernel path
    and the reference-layout launcher, replay, compare with the eager result"""
    s24 = mods["s24"]
    M, K, N = 512, 1024, 1024
    A = randn((M, K), torch.float16, 801).to(DEV)
    B = randn((K, N), torch.float16, 802).to(DEV)
    vals, E, tc = s24.prune_compress(A, want_ref=True, want_tc=True)
    eager = s24.spmm(vals, tc, B)
    eager2 = mods["two"].run_2_kernel_ws_matmul(A, B, tie="reference")
    assert torch.equal(eager, eager2)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            c1 = mods["two"].run_2_kernel_ws_matmul(A, B, tie="reference")
            c2 = mods["ws"].run_sparse_ws_matmul(vals, E, B, tune=False)
    torch.cuda.current_stream().wait_stream(side)
    c1.zero_()
    c2.zero_()
    g.replay()
    torch.cuda.synchronize()
    _status_ok(s24)
    assert torch.equal(c1, eager) and torch.equal(c2, eager)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 200, 384), (512, 1032, 1280), (1024, 2048, 4096)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [None, {"BM": 128, "BN": 128}, {"BM": 256, "BN": 128}, {"BM": 256, "BN": 256}, {"BM": 512, "BN": 224}])
def test_transposed_b_is_used_in_place(mods, M, N, K, dtype, cfg):
    """B passed as X.t() with X (N, K) row-major (activations stored (tokens, hidden)): the kernel
    reads X directly as a K-major operand; the result must equal the row-major-B product bit for bit"""
    s24 = mods["s24"]
    A, B, ap, vals, ml, e = _prepare(M, K, N, dtype, 300 + M + N + K)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    v = from_bits(vals, dtype, DEV)
    Bd = B.to(DEV)
    X = Bd.t().contiguous()                      # (N, K) row-major
    assert X.t().stride(0) == 1
    C_t = s24.spmm(v, tc, X.t(), manual_config=cfg)
    _status_ok(s24)
    _check(C_t, _reference(ap, B, dtype))
    C_n = s24.spmm(v, tc, Bd, manual_config=cfg)
    assert torch.equal(C_t, C_n)
    # padded rows (row stride > K) and the reference-layout metadata entry
    Xp = torch.zeros(N, K + 64, dtype=dtype, device=DEV)
    Xp[:, :K] = X
    E = torch.from_numpy(e).to(DEV)
    C_p = s24.spmm(v, E, Xp[:, :K].t(), meta_layout="ref", manual_config=cfg)
    assert torch.equal(C_p, C_n)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (384, 200, 512), (1024, 1032, 1024), (128, 8, 128)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_scatter_epilogue_writes_every_destination(mods, M, N, K, dtype):
    """s24_spmm_scatter on one GPU: three destinations (two blocks inside one wide buffer, one
    separate tensor) all receive the product, bit-identical to the plain kernel on the same tile,
    and nothing around the blocks is touched."""
    s24 = mods["s24"]
    A, B, ap, vals, ml, e = _prepare(M, K, N, dtype, 900 + M + N + K)
    tc = torch.from_numpy(oracle.meta_tc(ml, K).view(np.int32)).to(DEV)
    v, Bd = from_bits(vals, dtype, DEV), B.to(DEV)
    want = s24.spmm(v, tc, Bd, manual_config={"BM": 256, "BN": 256})
    ldc = 2 * N + 24
    wide = torch.full((M + 1, ldc), 3.0, dtype=dtype, device=DEV)
    other = torch.full((M, ldc), 5.0, dtype=dtype, device=DEV)
    dsts = [wide.data_ptr() + 2 * 8, wide.data_ptr() + 2 * (N + 16), other.data_ptr()]
    s24.spmm_scatter(v, tc, Bd, dsts, ldc)
    _status_ok(s24)
    assert torch.equal(wide[:M, 8:8 + N], want) and torch.equal(wide[:M, N + 16:2 * N + 16], want)
    assert torch.equal(other[:, :N], want)
    assert bool((wide[:, :8] == 3.0).all()) and bool((wide[:, 8 + N:N + 16] == 3.0).all())
    assert bool((wide[:, 2 * N + 16:] == 3.0).all()) and bool((wide[M] == 3.0).all())
    assert bool((other[:, N:] == 5.0).all())
    _check(want, _reference(ap, B, dtype))


@pytest.mark.parametrize("M,N,K", [(32, 16, 64), (160, 72, 192), (416, 256, 320)])
def test_partly_covered_tiles_through_the_reference_layout_entry(mods, M, N, K):
    """shapes that are multiples of 32 / 64 but not of 128, through run_sparse_ws_matmul(A_vals, E, B):
    the library converts E into a caller-sized workspace whose padding words it must make valid itself
    (the workspace is handed over full of an invalid code on purpose)"""
    s24 = mods["s24"]
    dtype = torch.float16
    A, B, ap, vals, ml, e = _prepare(M, K, N, dtype, 950 + M + N + K)
    v, E, Bd = from_bits(vals, dtype, DEV), torch.from_numpy(e).to(DEV), B.to(DEV)
    C = mods["ws"].run_sparse_ws_matmul(v, E, Bd)
    _status_ok(s24)
    ref32 = _reference(ap, B, dtype)
    _check(C, ref32)
    ws = torch.zeros((s24.meta_tc_numel(M, K),), dtype=torch.int32, device=DEV)   # code 0 is not a valid 2:4 code
    C2 = s24.spmm(v, E, Bd, meta_layout="ref", workspace=ws)
    _status_ok(s24)
    assert torch.equal(C, C2)
    assert np.array_equal(ws.cpu().numpy().view(np.uint32), oracle.meta_tc(ml, K))


def test_dense_baseline_module_is_importable_and_is_cublas(mods):
    """the reference's benchmark drivers import gluon_ws_dense beside gluon_ws_sparse; the stand-in
    is a cuBLAS product"""
    dense = load_dropin("gluon_ws_dense.py")
    A = randn((256, 512), torch.float16, 41).to(DEV)
    B = randn((512, 128), torch.float16, 42).to(DEV)
    C = dense.run_ws_matmul(A, B, tune=False, manual_config={"BM": 128})
    assert C.dtype == torch.float16 and torch.equal(C, A @ B)
