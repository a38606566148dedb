"""Import-compatible stand-in for compression/gluon_ws_dense.py (the reference's dense
warp-specialised GEMM, the "dense" line of its benchmarks: dev/8.11_benchmark_2_kernel.py:76).

The dense product is not part of the 2:4 path this library rebuilds; a plain dense GEMM is the
vendor library's job, so `run_ws_matmul` calls cuBLAS through `torch.matmul`.  It exists so that
the reference's benchmark drivers, which import this module next to `gluon_ws_sparse`, keep
working and keep their dense comparison line.
"""
import torch


def run_ws_matmul(A, B, tune=True, manual_config=None):
    """C = A @ B, freshly allocated in A's dtype (compression/gluon_ws_dense.py:477-520).
    `tune` and `manual_config` are accepted and ignored."""
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise RuntimeError(f"shapes do not chain: A {tuple(A.shape)}, B {tuple(B.shape)}")
    if not A.is_cuda or not B.is_cuda:
        raise RuntimeError("run_ws_matmul runs on CUDA tensors only")
    return torch.matmul(A, B)
