"""Generate the golden vectors under tests/golden from the reference's own Python code.

Run where the reference project is checked out, passing its root:

    python tests/golden/make_golden.py <reference_root>

It imports the reference's ``compression/prune.py`` and ``compression/compress_2_4.py``
unmodified, runs them on CPU on seeded inputs and stores inputs + outputs as raw 16-bit
patterns.  It also measures how the reference's ``torch.topk`` breaks ties and writes
that as a 729-entry weak-ordering table to

    tests/golden/tie_table.json     (the fixture)
    oracle/tie_table.inc            (read by the CPU oracle)

tests/test_oracle_golden.py checks that the two copies agree; the CUDA library states the
same behaviour as a rule (csrc/prune_core.cuh, keep_mask_scalar) which
tests/test_prune_core_host.py checks against the table for all 75 weak orderings.
"""
import itertools
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py <reference_root>")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "compression"))

from prune import prune_2_4  # noqa: E402  (reference)
from compress_2_4 import compress_dense_to_sparse, _calculate_meta_reordering_offsets  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def weak_index(k):
    idx, mul = 0, 1
    for i in range(4):
        for j in range(i + 1, 4):
            t = 0 if k[i] < k[j] else (1 if k[i] == k[j] else 2)
            idx += t * mul
            mul *= 3
    return idx


def measure_tie_table():
    pats = list(itertools.product([1.0, 2.0, 3.0, 4.0], repeat=4))  # no zeros: mask readable from != 0
    table = np.full(729, 0xFF, dtype=np.uint8)
    for dtype in (torch.float16, torch.bfloat16, torch.float32):
        for shape in ((256, 4), (1, 1024), (32, 32)):
            x = torch.tensor(pats, dtype=torch.float32).to(dtype).reshape(shape)
            kept = (prune_2_4(x) != 0).reshape(256, 4)
            assert (kept.sum(1) == 2).all()
            for p, k in zip(pats, kept.tolist()):
                m = sum(1 << i for i in range(4) if k[i])
                w = weak_index(p)
                assert table[w] in (0xFF, m), "tie behaviour is not a function of the weak ordering"
                table[w] = m
    assert int((table != 0xFF).sum()) == 75
    return table


def case(name, A, dtype):
    """Run the reference on A (float32 tensor cast to dtype) and collect everything."""
    A = A.to(dtype)
    M, K = A.shape
    pruned = prune_2_4(A)
    vals, meta = compress_dense_to_sparse(pruned)
    E = meta.view(M // 16, K)
    mag_mask = prune_2_4(A.abs()) != 0
    pruned_mag = torch.where(mag_mask, A, torch.zeros_like(A))  # masked_fill semantics, prune.py:91
    vals_mag, meta_mag = compress_dense_to_sparse(pruned_mag)
    return {
        f"{name}.A": bits(A),
        f"{name}.pruned": bits(pruned),
        f"{name}.vals": bits(vals),
        f"{name}.E": E.contiguous().numpy().copy(),
        f"{name}.pruned_mag": bits(pruned_mag),
        f"{name}.vals_mag": bits(vals_mag),
        f"{name}.E_mag": meta_mag.view(M // 16, K).contiguous().numpy().copy(),
    }


def main():
    table = measure_tie_table()
    inc = ",\n".join(", ".join(str(int(v)) for v in table[i:i + 27]) for i in range(0, 729, 27)) + "\n"
    (ROOT / "oracle" / "tie_table.inc").write_text(inc)
    (HERE / "tie_table.json").write_text(json.dumps({
        "source": "compression/prune.py:85 torch.topk(k=2, largest=False) on CPU, torch " + torch.__version__,
        "index": "sum over pairs (01,02,03,12,13,23) of t*3^p, t=0 if k_i<k_j, 1 if equal, 2 if greater",
        "value": "keep mask, bit i = element i survives; 255 = inconsistent ordering",
        "table": [int(v) for v in table],
    }))

    out = {}
    g = torch.Generator().manual_seed(20240611)
    # random N(0,1) like every reference self-check (gluon_ws_sparse.py:651-652)
    out.update(case("randn_f16", torch.randn(64, 128, generator=g), torch.float16))
    out.update(case("randn_bf16", 0.02 * torch.randn(32, 192, generator=g), torch.bfloat16))
    # tie-heavy: tiny alphabet with negatives, zeros and -0.0 so that every weak ordering,
    # kept zeros and all-zero groups occur
    alpha = torch.tensor([-2.0, -1.0, -0.0, 0.0, 0.0, 1.0, 1.0, 2.0])
    idx = torch.randint(0, len(alpha), (96, 256), generator=g)
    out.update(case("ties_f16", alpha[idx], torch.float16))
    idx = torch.randint(0, len(alpha), (32, 64), generator=g)
    out.update(case("ties_bf16", alpha[idx], torch.bfloat16))
    # special values: infinities, largest finite, subnormals
    spec = torch.tensor([float("inf"), -float("inf"), 65504.0, -65504.0, 6e-8, -6e-8, 1e-5, 0.0, -0.0, 1.0])
    idx = torch.randint(0, len(spec), (32, 64), generator=g)
    out.update(case("special_f16", spec[idx], torch.float16))

    # encoder table (compress_2_4.py:79-104): arbitrary non-zero patterns, not 2:4
    flags = torch.randint(0, 2, (64, 128), generator=g).float()
    dense = (flags * (1.0 + torch.rand(64, 128, generator=g))).to(torch.float16)
    v, m = compress_dense_to_sparse(dense)
    out["flags_f16.dense"] = bits(dense)
    out["flags_f16.vals"] = bits(v)
    out["flags_f16.E"] = m.view(4, 128).contiguous().numpy().copy()

    for (m_, nc) in ((32, 4), (64, 8), (128, 16)):
        out[f"offsets_{m_}_{nc}"] = _calculate_meta_reordering_offsets(m_, nc, "cpu").numpy().copy()

    # GEMM: expected = A_pruned @ B (gluon_ws_sparse.py:660) with fp32 accumulation
    A = torch.randn(128, 256, generator=g).to(torch.float16)
    B = torch.randn(256, 64, generator=g).to(torch.float16)
    Ap = prune_2_4(A)
    out["gemm_f16.A"] = bits(A)
    out["gemm_f16.B"] = bits(B)
    out["gemm_f16.C_f32"] = (Ap.float() @ B.float()).numpy().copy()
    out["gemm_f16.C"] = bits((Ap.float() @ B.float()).to(torch.float16))

    np.savez_compressed(HERE / "golden.npz", **out)
    print("wrote", HERE / "golden.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
