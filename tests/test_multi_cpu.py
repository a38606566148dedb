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
    assert row_panels(160, 4) == [(0, 128), (128, 160)]            # ragged tail stays in the last panel
    assert row_panels(96, 4) == [(0, 96)]
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


# ---------------------------------------------------------------- replicated="fused" on CPU ranks

_KEY = 1 << 40   # fake device addresses: key * 2^40 + byte offset


class _FileBackend:
    """Stand-in for the CUDA IPC helpers: each "allocation" is a file mapped shared, so a rank's
    stores into a peer's buffer really land in the peer process."""

    def __init__(self, directory, rank):
        self.dir, self.rank, self.maps, self.n = directory, rank, {}, 0

    def _map(self, name, nbytes):
        key = len(self.maps) + 1
        self.maps[key] = torch.from_file(os.path.join(self.dir, name), shared=True, size=nbytes // 2, dtype=torch.int16)
        return key * _KEY

    def alloc(self, nbytes):
        self.n += 1
        name = f"r{self.rank}_{self.n}"
        with open(os.path.join(self.dir, name), "wb") as f:
            f.truncate(nbytes)
        ptr = self._map(name, nbytes)
        self.names = getattr(self, "names", {})
        self.names[ptr] = (name, nbytes)
        return ptr

    def export(self, ptr):
        name, nbytes = self.names[ptr]
        return f"{name}:{nbytes}".encode().ljust(64, b"\0")

    def open(self, handle):
        name, nbytes = handle.rstrip(b"\0").decode().split(":")
        return self._map(name, int(nbytes))

    def close(self, ptr):
        self.maps.pop(ptr // _KEY)

    def free(self, ptr):
        self.maps.pop(ptr // _KEY)

    def as_tensor(self, ptr, rows, cols, dtype):
        return self.maps[ptr // _KEY].view(dtype).view(rows, cols)

    def copy_2d(self, dst, dst_pitch, src, src_pitch, width_bytes, rows, stream):
        """pitched block copy between two mapped files (what the copy engines do between GPUs)"""
        dk, doff = divmod(dst, _KEY)
        sk, soff = divmod(src, _KEY)
        d = self.maps[dk].view(torch.uint8)
        s_ = self.maps[sk].view(torch.uint8)
        for r in range(rows):
            d[doff + r * dst_pitch:doff + r * dst_pitch + width_bytes] = s_[soff + r * src_pitch:soff + r * src_pitch + width_bytes]


def _fused_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=__import__("datetime").timedelta(seconds=30))
    try:
        backend = _FileBackend(result_dir, rank)

        def fake_scatter(vals, meta_tc, B, dst_ptrs, ldc):
            C = (vals.float() @ B.float()).to(vals.dtype)
            for ptr in dst_ptrs:
                key, off = divmod(ptr, _KEY)
                flat = backend.maps[key].view(vals.dtype)
                rows = flat.numel() // ldc
                col0 = (off // 2) % ldc
                assert off // 2 < ldc                      # the offset is a column of row 0
                flat.view(rows, ldc)[:, col0:col0 + B.shape[1]] = C

        torch.manual_seed(11)
        M, K, N = 256, 128, 32 * world
        A = torch.randn(M, K).to(torch.bfloat16)
        op = NShardedSpmm(A, torch.zeros(1, dtype=torch.int32), scatter_fn=fake_scatter, peer_backend=backend)
        op.K = K
        n0, n1 = op.local_columns(N)
        for it in range(3):                                # the result buffer is reused call after call
            B = torch.randn(K, N).to(torch.bfloat16)
            want = (A.float() @ B.float()).to(torch.bfloat16)
            C = op(B[:, n0:n1].contiguous(), n_total=N, replicated="fused")
            assert C.shape == (M, N) and C.dtype == torch.bfloat16
            assert torch.equal(C, want), f"iteration {it}"
        assert len(op._peer.ptrs) == world and op._peer.ptrs[rank] == op._peer._own
        # replicated="copy": the product lands in this rank's copy in row panels, each pushed to the peers as a
        # pitched block; same buffer, same fences
        def fake_spmm(vals, meta_tc, Bs, out=None):
            c = (vals.float() @ Bs.float()).to(vals.dtype)
            if out is None:
                return c
            out.copy_(c)
            return out
        op.spmm_fn = fake_spmm
        op._meta_rows = lambda r0, r1: None
        for it in range(2):
            B = torch.randn(K, N).to(torch.bfloat16)
            want = (A.float() @ B.float()).to(torch.bfloat16)
            C = op(B[:, n0:n1].contiguous(), n_total=N, replicated="copy", panels=2)
            assert torch.equal(C, want), f"copy mode, iteration {it}"
        op.close()
        assert op._peer is None and not backend.maps       # every mapping released
        with open(os.path.join(result_dir, f"fused_ok_{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_fused_replicated_result_through_peer_buffers(tmp_path, world):
    mp.spawn(_fused_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"fused_ok_{r}").exists() for r in range(world))
