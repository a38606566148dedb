"""Helpers shared by the GPU parity tests: bit-level views and oracle wrappers."""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "gpu-compression-kernel_b200"
DROPIN = PKG / "compression"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)

import oracle  # noqa: E402

ODT = {torch.float16: oracle.FP16, torch.bfloat16: oracle.BF16}
MODE = {"signed": oracle.MODE_SIGNED, "magnitude": oracle.MODE_MAGNITUDE}
TIE = {"reference": oracle.TIE_REFERENCE, "lower": oracle.TIE_LOWER, "higher": oracle.TIE_HIGHER}


def bits(t: torch.Tensor) -> np.ndarray:
    """raw 16-bit patterns of an fp16 / bf16 tensor as a uint16 numpy array (on CPU)"""
    return t.detach().contiguous().cpu().view(torch.int16).numpy().view(np.uint16)


def from_bits(a: np.ndarray, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(dtype).to(device)


def randn(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(dtype)


def tie_heavy(shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    alpha = torch.tensor([-2.0, -1.0, -0.0, 0.0, 0.5, 1.0, 1.0, 2.0])
    return alpha[torch.randint(0, len(alpha), shape, generator=g)].to(dtype)


def load_dropin(name: str):
    """import a drop-in module flat from the `compression` directory (the way the
    reference's scripts import theirs) or, for the numbered kernel files, by path"""
    import importlib.util
    path = DROPIN / name
    spec = importlib.util.spec_from_file_location("dropin_" + path.stem.replace(".", "_"), path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
