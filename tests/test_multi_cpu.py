"""Host logic of the N-sharded multi-GPU path on CPU ranks (gloo, world size 2).

The product has no CPU GEMM, so the ranks get a stand-in product (dense torch matmul of a
decompressed A) through NShardedSpmm's `spmm_fn` hook: what is tested here is the sharding
arithmetic, the panel-wise all-gather and its re-layout, and that a failing rank surfaces as
an error on the others instead of a hang.
"""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "gpu-compression-kernel_b200"))

from s24.multi import NShardedSpmm, row_panels, shard_bounds  # noqa: E402


def test_shard_bounds_cover_and_align():
    for n, world in [(8192, 8), (65536, 8), (200, 3), (1032, 4), (8, 8), (16, 3)]:
        prev = 0
        for r in range(world):
            a, b = shard_bounds(n, world, r)
            assert a == prev and a % 8 == 0 and b % 8 == 0 and b >= a
            prev = b
        assert prev == n
    with pytest.raises(ValueError):
        shard_bounds(100, 2, 0)
    with pytest.raises(ValueError):
        shard_bounds(64, 2, 2)


def test_row_panels():
    assert row_panels(1024, 4) == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    assert row_panels(384, 4) == [(0, 128), (128, 256), (256, 384)]
    assert row_panels(28672, 8)[-1][1] == 28672
    assert all((b - a) % 128 == 0 for a, b in row_panels(28672, 8))
    with pytest.raises(ValueError):
        row_panels(100, 2)


def _fake_spmm(dense_by_ptr):
    """stand-in for the GPU kernel: `vals` is a dense float A here, metadata is ignored"""
    def fn(vals, meta_tc, B, out=None):
        return vals @ B
    return fn


def _worker(rank, world, port, fail_rank, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=20))
    try:
        torch.manual_seed(7)
        M, K, N = 384, 256, 64 * world
        A = torch.randn(M, K)
        B = torch.randn(K, N)
        # vals stands in for the compressed operand; K/2 columns are what NShardedSpmm sizes K from
        op = NShardedSpmm(A, torch.zeros((M // 128) * (K // 128) * 512, dtype=torch.int32), spmm_fn=_fake_spmm(None))
        op.K = K                                   # dense stand-in: K is not 2 * vals.shape[1]
        n0, n1 = op.local_columns(N)
        assert (n1 - n0) == N // world
        if rank == fail_rank:
            raise RuntimeError("injected failure on this rank before its collective")
        C_local = op(B[:, n0:n1].contiguous())
        assert torch.allclose(C_local, (A @ B)[:, n0:n1], atol=1e-5)
        C_full = op(B[:, n0:n1].contiguous(), n_total=N, replicated=True, panels=3)
        assert C_full.shape == (M, N)
        assert torch.allclose(C_full, A @ B, atol=1e-5)
        torch.save(C_full, os.path.join(result_dir, f"c_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_ranks_shard_and_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), -1, str(tmp_path)), nprocs=world, join=True)
    c0 = torch.load(tmp_path / "c_0.pt")
    c1 = torch.load(tmp_path / "c_1.pt")
    assert torch.equal(c0, c1)                     # replicated result is identical on both ranks


def test_failing_rank_is_an_error_not_a_hang(tmp_path):
    """failure injected on the host: rank 1 raises before its collective; rank 0's all-gather
    must end with an error within the process-group timeout"""
    world = 2
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(world, _free_port(), 1, str(tmp_path)), nprocs=world, join=True)
