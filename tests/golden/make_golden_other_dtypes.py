"""Golden vectors for the element types of compress_dense_to_sparse beyond fp16 / bf16.

    python tests/golden/make_golden_other_dtypes.py <reference_root>

Imports the reference's ``compression/compress_2_4.py`` unmodified and runs it on CPU on seeded
inputs of its three other branches (compress_2_4.py:41-47,73-76,144-154): int8 (2:4, int32
metadata of eight codes), int32 (2:4, int16 metadata) and float32 (1:2, int16 metadata).
Inputs and outputs are stored raw in tests/golden/golden_other_dtypes.npz.
"""
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden_other_dtypes.py <reference_root>")
sys.path.insert(0, str(Path(sys.argv[1]) / "compression"))

from compress_2_4 import compress_dense_to_sparse  # noqa: E402  (reference)


def main():
    g = torch.Generator().manual_seed(20250101)
    out = {}
    # arbitrary non-zero patterns (not only 2:4 / 1:2), so every row of the encoder table occurs
    for name, dtype, shape in (("int8", torch.int8, (48, 256)), ("int32", torch.int32, (64, 128)),
                               ("float32", torch.float32, (32, 96))):
        flags = torch.randint(0, 2, shape, generator=g)
        mag = torch.randint(1, 100, shape, generator=g) * (1 - 2 * torch.randint(0, 2, shape, generator=g))
        dense = (flags * mag).to(dtype)
        if dtype == torch.float32:
            dense = dense * 0.37
            dense[0, :8] = torch.tensor([0.0, -0.0, -0.0, 1.5, -0.0, -0.0, 0.0, 0.0])   # signed zeros count as zero
        vals, meta = compress_dense_to_sparse(dense)
        out[f"{name}.dense"] = dense.numpy().copy()
        out[f"{name}.vals"] = vals.contiguous().numpy().copy()
        out[f"{name}.meta"] = meta.contiguous().numpy().copy()
    np.savez_compressed(HERE / "golden_other_dtypes.npz", **out)
    print({k: (v.shape, v.dtype) for k, v in out.items()})


if __name__ == "__main__":
    main()
