"""Drop-in for the reference's compression/prune.py: same names, arguments, return values
and error behaviour; `prune_2_4` runs on the B200 through libs24 (C ABI `s24_prune`).

`gen_mask` / `prune_tensor` are not on any timed path of the reference; they are kept as
small torch utilities so that `from prune import *` keeps working.
"""
import torch

import sys
from pathlib import Path

_PKG_ROOT = str(Path(__file__).resolve().parent.parent)   # makes `s24` importable however this file is loaded
if _PKG_ROOT not in sys.path:
    sys.path.insert(0, _PKG_ROOT)
import s24  # noqa: E402


def gen_mask(device: torch.device, size: tuple, n: int, m: int):
    """Random pattern with n ones among m positions, tiled `size` times
    (compression/prune.py:3-29)."""
    if n > m:
        raise ValueError("n cannot be greater than m.")
    pattern = torch.zeros(m, dtype=torch.int32, device=device)
    pattern[torch.randperm(m, device=device)[:n]] = 1
    return pattern.repeat(size)


def prune_tensor(x: torch.Tensor, n: int = 2, m: int = 4):
    """Multiply x in place by a random fixed n:m pattern (compression/prune.py:31-55)."""
    assert len(x.shape) == 2, "The tensor must be 2-dimensional"
    assert x.shape[1] % m == 0, "The tensor's second dimension must be divisible by the values of m"
    x *= gen_mask(x.device, size=(x.shape[0], x.shape[1] // m), n=n, m=m)
    return x


def prune_2_4(tensor: torch.Tensor, mode: str = "signed", tie: str = "reference") -> torch.Tensor:
    """For each contiguous group of 4 along the last dimension set the two smallest values
    to 0 and return a new tensor (compression/prune.py:57-96).

    Defaults reproduce the reference bit for bit, including how its `torch.topk` breaks
    ties.  `mode="magnitude"` ranks by |x|; `tie="lower"` / `"higher"` pick a fixed rule.
    Raises ValueError if the last dimension is not divisible by 4.
    """
    if tensor.size(-1) % 4 != 0:
        raise ValueError("The size of the last dimension must be divisible by 4.")
    return s24.prune(tensor, mode=mode, tie=tie)
