"""The packed bit logic of the CUDA prune/compress kernels, compiled for the host.

csrc/prune_core.cuh is host+device; here g++ builds it into a small shared object and
every result is compared bit for bit with the oracle (which is itself pinned to the
reference's outputs).  This checks the arithmetic the GPU kernels execute without needing
a GPU; the kernels' memory indexing is covered by the `gpu` tests.
"""
import ctypes
import itertools
import subprocess
from pathlib import Path

import numpy as np
import pytest

import oracle

ROOT = Path(__file__).resolve().parent.parent
SRC = ROOT / "tests/host/prune_core_host.cpp"
INC = ROOT / "gpu-compression-kernel_b200/csrc"


@pytest.fixture(scope="module")
def host(tmp_path_factory):
    so = tmp_path_factory.mktemp("host") / "libprune_core_host.so"
    subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-x", "c++", f"-I{INC}", str(SRC), "-o", str(so)],
                   check=True)
    L = ctypes.CDLL(str(so))
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.host_prune_compress.argtypes = [vp, i64, i64, i32, i32, i32, vp, vp]
    L.host_prune.argtypes = [vp, i64, i32, i32, i32, vp]
    L.host_prune_compress_from_mask.argtypes = [vp, i64, i64, i32, vp, vp]
    L.host_keep_mask.argtypes = [vp, i32]
    L.host_keep_mask.restype = ctypes.c_uint
    return L


def _pc(host, a, dtype, mode, tie):
    a = np.ascontiguousarray(a)
    M, K = a.shape
    vals = np.zeros((M, K // 2), np.uint16)
    meta = np.zeros((M, K // 16), np.uint16)
    host.host_prune_compress(a.ctypes.data, M, K, dtype, mode, tie, vals.ctypes.data, meta.ctypes.data)
    return vals, meta.view(np.int16)


def _p(host, a, dtype, mode, tie):
    a = np.ascontiguousarray(a)
    out = np.zeros_like(a)
    host.host_prune(a.ctypes.data, a.size, dtype, mode, tie, out.ctypes.data)
    return out


def test_reference_tie_rule_equals_measured_table(host):
    tt = oracle.tie_table()
    L = oracle.lib()
    seen = set()
    for p in itertools.product([1.0, 2.0, 3.0, 4.0], repeat=4):
        k = np.array(p, dtype=np.float32)
        w = L.s24o_weak_order_index(k.ctypes.data)
        seen.add(w)
        assert host.host_keep_mask(k.ctypes.data, 0) == tt[w], p
    assert len(seen) == 75


def _alphabet_matrix(dtype_np_bits, alphabet_bits, M, K, seed):
    rng = np.random.default_rng(seed)
    return np.asarray(alphabet_bits, dtype=np.uint16)[rng.integers(0, len(alphabet_bits), size=(M, K))]


F16 = {"-2": 0xC000, "-1": 0xBC00, "-0": 0x8000, "0": 0x0000, "1": 0x3C00, "2": 0x4000, "inf": 0x7C00,
       "-inf": 0xFC00, "sub": 0x0001, "-sub": 0x8001, "max": 0x7BFF}
BF16 = {"-2": 0xC000, "-1": 0xBF80, "-0": 0x8000, "0": 0x0000, "1": 0x3F80, "2": 0x4000, "inf": 0x7F80,
        "-inf": 0xFF80, "sub": 0x0001, "-sub": 0x8001, "max": 0x7F7F}


@pytest.mark.parametrize("dtype,alpha", [(oracle.FP16, F16), (oracle.BF16, BF16)])
@pytest.mark.parametrize("mode", [oracle.MODE_SIGNED, oracle.MODE_MAGNITUDE])
@pytest.mark.parametrize("tie", [oracle.TIE_REFERENCE, oracle.TIE_LOWER, oracle.TIE_HIGHER])
def test_tie_heavy_alphabet(host, dtype, alpha, mode, tie):
    a = _alphabet_matrix(np.uint16, list(alpha.values()), 64, 256, seed=dtype * 10 + mode * 3 + tie)
    want_p = oracle.prune(a, dtype, mode, tie)
    want_v, want_ml, _ = oracle.compress(want_p, dtype)
    got_v, got_ml = _pc(host, a, dtype, mode, tie)
    assert np.array_equal(got_v, want_v)
    assert np.array_equal(got_ml, want_ml)
    assert np.array_equal(_p(host, a, dtype, mode, tie), want_p)


@pytest.mark.parametrize("dtype", [oracle.FP16, oracle.BF16])
def test_all_256_four_symbol_patterns(host, dtype):
    sym = [0x0000, 0x3C00, 0xBC00, 0x4000] if dtype == oracle.FP16 else [0x0000, 0x3F80, 0xBF80, 0x4000]
    pats = np.array(list(itertools.product(sym, repeat=4)), dtype=np.uint16)      # (256, 4)
    a = np.tile(pats.reshape(16, 64), (2, 1))                                      # (32, 64)
    for mode in (oracle.MODE_SIGNED, oracle.MODE_MAGNITUDE):
        want_p = oracle.prune(a, dtype, mode, oracle.TIE_REFERENCE)
        want_v, want_ml, _ = oracle.compress(want_p, dtype)
        got_v, got_ml = _pc(host, a, dtype, mode, oracle.TIE_REFERENCE)
        assert np.array_equal(got_v, want_v) and np.array_equal(got_ml, want_ml)


@pytest.mark.parametrize("name,dtype", [("randn_f16", oracle.FP16), ("randn_bf16", oracle.BF16),
                                        ("ties_f16", oracle.FP16), ("ties_bf16", oracle.BF16),
                                        ("special_f16", oracle.FP16)])
def test_golden_inputs(host, golden, name, dtype):
    a = golden[f"{name}.A"]
    M, K = a.shape
    got_v, got_ml = _pc(host, a, dtype, oracle.MODE_SIGNED, oracle.TIE_REFERENCE)
    assert np.array_equal(got_v, golden[f"{name}.vals"])
    off = oracle.meta_offsets(M, K // 16)
    assert np.array_equal(got_ml, golden[f"{name}.E"].reshape(-1)[off].reshape(M, K // 16))
    assert np.array_equal(_p(host, a, dtype, oracle.MODE_SIGNED, oracle.TIE_REFERENCE), golden[f"{name}.pruned"])


def test_compress_only_mode_matches_encoder_table(host, golden):
    d = golden["flags_f16.dense"]
    got_v, got_ml = _pc(host, d, oracle.FP16, 2, oracle.TIE_REFERENCE)   # mode 2 = no pruning
    want_v, want_ml, _ = oracle.compress(d, oracle.FP16)
    assert np.array_equal(got_v, want_v) and np.array_equal(got_ml, want_ml)
    assert np.array_equal(got_v, golden["flags_f16.vals"])


def test_random_bits_no_nan(host):
    rng = np.random.default_rng(99)
    a = rng.integers(0, 65536, size=(64, 512), dtype=np.uint16)
    for dtype, expmask in ((oracle.FP16, 0x7C00), (oracle.BF16, 0x7F80)):
        b = a.copy()
        nan = ((b & expmask) == expmask) & ((b & (~expmask & 0x7FFF)) != 0)
        b[nan] = 0x3C00                                   # NaN inputs are unsupported
        for mode in (0, 1):
            want_p = oracle.prune(b, dtype, mode, 0)
            want_v, want_ml, _ = oracle.compress(want_p, dtype)
            got_v, got_ml = _pc(host, b, dtype, mode, 0)
            assert np.array_equal(got_v, want_v) and np.array_equal(got_ml, want_ml)
            assert np.array_equal(_p(host, b, dtype, mode, 0), want_p)


@pytest.mark.parametrize("dtype,alpha", [(oracle.FP16, F16), (oracle.BF16, BF16)])
def test_epilogue_variant_encodes_from_the_keep_mask(host, dtype, alpha):
    """prune_compress_8_from_mask (the GEMM's pruning epilogue): the keep mask is the oracle's signed,
    lower-index prune, and the codes name the kept positions even where a kept value is an exact zero
    (compression/kernels/10.1_prune_acc.py:115-117 encodes from its mask)"""
    rng = np.random.default_rng(5 + dtype)
    tie_heavy = _alphabet_matrix(np.uint16, [v for k, v in alpha.items()], 64, 256, seed=17 + dtype)
    rand = rng.integers(0, 65536, size=(64, 256), dtype=np.uint16)
    expmask = 0x7C00 if dtype == oracle.FP16 else 0x7F80
    nan = ((rand & expmask) == expmask) & ((rand & (~expmask & 0x7FFF)) != 0)
    rand[nan] = 0x3C00
    for a in (tie_heavy, rand):
        a = np.ascontiguousarray(a)
        M, K = a.shape
        vals = np.zeros((M, K // 2), np.uint16)
        meta = np.zeros((M, K // 16), np.uint16)
        host.host_prune_compress_from_mask(a.ctypes.data, M, K, dtype, vals.ctypes.data, meta.ctypes.data)
        _, want_mask = oracle.prune(a, dtype, oracle.MODE_SIGNED, oracle.TIE_LOWER, return_mask=True)
        w = meta.astype(np.uint32)
        codes = np.stack([(w >> (4 * j)) & 0xF for j in range(4)], axis=-1).reshape(M, K // 4)
        idx0, idx1 = codes & 3, codes >> 2
        assert (idx0 < idx1).all()
        got_mask = ((1 << idx0) | (1 << idx1)).astype(np.uint8)
        assert np.array_equal(got_mask, want_mask)
        groups = a.reshape(M, K // 4, 4)
        v = vals.reshape(M, K // 4, 2)
        assert np.array_equal(v[..., 0], np.take_along_axis(groups, idx0[..., None].astype(np.int64), -1)[..., 0])
        assert np.array_equal(v[..., 1], np.take_along_axis(groups, idx1[..., None].astype(np.int64), -1)[..., 0])
