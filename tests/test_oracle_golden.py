"""The CPU oracle against the reference's own outputs (tests/golden/golden.npz).

The fixtures were produced by the reference's prune_2_4 / compress_dense_to_sparse
(compression/prune.py:57-96, compression/compress_2_4.py:32-161); every comparison here is
bit-exact.
"""
import itertools
import json
from pathlib import Path

import numpy as np
import pytest

import oracle

ROOT = Path(__file__).resolve().parent.parent
CASES = [("randn_f16", oracle.FP16), ("randn_bf16", oracle.BF16), ("ties_f16", oracle.FP16),
         ("ties_bf16", oracle.BF16), ("special_f16", oracle.FP16)]


def test_tie_table_copies_agree():
    fixture = np.array(json.loads((ROOT / "tests/golden/tie_table.json").read_text())["table"], dtype=np.uint8)
    assert np.array_equal(oracle.tie_table(), fixture)
    assert int((fixture != 0xFF).sum()) == 75          # number of weak orderings of 4 keys
    for m in fixture[fixture != 0xFF]:
        assert bin(int(m)).count("1") == 2


def test_tie_table_only_differs_from_lower_rule_where_index0_is_smallest():
    # documents the artefact: of the 75 orderings the reference departs from
    # "lower index wins" only when element 0 is the strict minimum and the tie is among 1..3
    tt = oracle.tie_table()
    L = oracle.lib()
    diff = 0
    for p in itertools.product([1.0, 2.0, 3.0, 4.0], repeat=4):
        k = np.array(p, dtype=np.float32)
        w = L.s24o_weak_order_index(k.ctypes.data)
        order = sorted(range(4), key=lambda i: (-p[i], i))
        lower = (1 << order[0]) | (1 << order[1])
        if tt[w] != lower:
            diff += 1
            assert p[0] < min(p[1:])
    assert diff == 18


@pytest.mark.parametrize("name,dtype", CASES)
def test_prune_matches_reference(golden, name, dtype):
    got = oracle.prune(golden[f"{name}.A"], dtype, oracle.MODE_SIGNED, oracle.TIE_REFERENCE)
    assert np.array_equal(got, golden[f"{name}.pruned"])
    got = oracle.prune(golden[f"{name}.A"], dtype, oracle.MODE_MAGNITUDE, oracle.TIE_REFERENCE)
    # magnitude variant: keep mask = prune_2_4(|A|) != 0 (the reference's code on |A|)
    assert np.array_equal(got, golden[f"{name}.pruned_mag"])


@pytest.mark.parametrize("name,dtype", CASES)
def test_compress_matches_reference(golden, name, dtype):
    vals, ml, mr = oracle.compress(golden[f"{name}.pruned"], dtype)
    assert np.array_equal(vals, golden[f"{name}.vals"])
    assert np.array_equal(mr, golden[f"{name}.E"])
    M, K = golden[f"{name}.pruned"].shape
    off = oracle.meta_offsets(M, K // 16)
    assert np.array_equal(mr.reshape(-1)[off].reshape(M, K // 16), ml)
    # fused call used by the CPU baseline
    v2, e2 = oracle.prune_compress(golden[f"{name}.A"], dtype)
    assert np.array_equal(v2, vals) and np.array_equal(e2, mr)


@pytest.mark.parametrize("name,dtype", CASES)
def test_compress_magnitude_metadata(golden, name, dtype):
    pm = oracle.prune(golden[f"{name}.A"], dtype, oracle.MODE_MAGNITUDE)
    vals, ml, mr = oracle.compress(pm, dtype)
    assert np.array_equal(mr, golden[f"{name}.E_mag"])
    assert np.array_equal(vals, golden[f"{name}.vals_mag"])


def test_encoder_table_all_flag_patterns(golden):
    # arbitrary non-zero patterns, including fewer and more than two per group
    vals, ml, mr = oracle.compress(golden["flags_f16.dense"], oracle.FP16)
    assert np.array_equal(vals, golden["flags_f16.vals"])
    assert np.array_equal(mr, golden["flags_f16.E"])
    codes = set()
    for w in ml.reshape(-1).astype(np.uint16):
        codes.update((int(w) >> s) & 0xF for s in (0, 4, 8, 12))
    assert codes <= {4, 8, 9, 12, 13, 14}


@pytest.mark.parametrize("m,nc", [(32, 4), (64, 8), (128, 16)])
def test_meta_offsets(golden, m, nc):
    assert np.array_equal(oracle.meta_offsets(m, nc), golden[f"offsets_{m}_{nc}"])


def test_gemm_f32acc(golden):
    ap = oracle.prune(golden["gemm_f16.A"], oracle.FP16)
    c32, c16 = oracle.gemm_f32acc(ap, golden["gemm_f16.B"], oracle.FP16)
    np.testing.assert_allclose(c32, golden["gemm_f16.C_f32"], rtol=1e-5, atol=1e-4)
    got = c16.view(np.float16).astype(np.float32)
    ref = golden["gemm_f16.C"].view(np.float16).astype(np.float32)
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2)


def test_decompress_round_trip(golden):
    pr = golden["randn_f16.pruned"]
    vals, ml, _ = oracle.compress(pr, oracle.FP16)
    assert np.array_equal(oracle.decompress(vals, ml), pr)


def test_meta_tc_layout_is_a_permutation_of_row_pairs():
    rng = np.random.default_rng(5)
    M, K = 256, 384
    ml = rng.integers(-32768, 32767, size=(M, K // 16), dtype=np.int16)
    tc = oracle.meta_tc(ml, K).reshape(M // 128, K // 128, 128, 4)
    u = ml.view(np.uint16).astype(np.uint32)
    for t, kb, L, j in [(0, 0, 0, 0), (1, 2, 77, 3), (0, 1, 127, 2), (1, 0, 8, 1)]:
        m0, k1, m2 = L % 8, (L // 8) % 2, L // 16
        r, c = 128 * t + 16 * m2 + m0, 8 * kb + 2 * j + k1
        assert tc[t, kb, L, j] == (u[r, c] | (u[r + 8, c] << 16))


def test_error_behaviour():
    a = np.zeros((32, 66), dtype=np.uint16)
    with pytest.raises(ValueError):
        oracle.prune(a)
    with pytest.raises(RuntimeError):
        oracle.compress(np.zeros((16, 64), dtype=np.uint16))
    with pytest.raises(RuntimeError):
        oracle.compress(np.zeros((32, 40), dtype=np.uint16))
    with pytest.raises(AssertionError):
        oracle.compress(np.zeros((32, 48), dtype=np.uint16))


@pytest.mark.parametrize("name", ["int8", "int32", "float32"])
def test_other_element_types_match_the_reference(name):
    """compress_dense_to_sparse's int8 / int32 / float32 branches (compress_2_4.py:41-47,73-76,144-154):
    the oracle against outputs of the reference's own function (tests/golden/make_golden_other_dtypes.py)"""
    import numpy as np
    from pathlib import Path
    g = dict(np.load(Path(__file__).resolve().parent / "golden" / "golden_other_dtypes.npz"))
    vals, meta = oracle.compress_other(g[f"{name}.dense"])
    assert vals.dtype == g[f"{name}.vals"].dtype and meta.dtype == g[f"{name}.meta"].dtype
    assert np.array_equal(vals.view(np.uint8), g[f"{name}.vals"].view(np.uint8))      # bit patterns, -0.0 included
    assert np.array_equal(meta, g[f"{name}.meta"])


def test_other_element_types_reject_what_the_reference_rejects():
    import numpy as np
    with pytest.raises(RuntimeError, match="divisible by 16"):
        oracle.compress_other(np.zeros((8, 128), np.int8))
    with pytest.raises(RuntimeError, match="divisible by 32"):
        oracle.compress_other(np.zeros((16, 48), np.int8))
    with pytest.raises(RuntimeError, match="divisible by 32"):
        oracle.compress_other(np.zeros((16, 64), np.float32))
    with pytest.raises(AssertionError):
        oracle.compress_other(np.zeros((32, 16), np.float32))     # 2 metadata columns
