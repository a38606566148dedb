"""N-sharded sparse GEMM across the GPUs of one box (one process per GPU).

C[:, n0:n1] = A24 . B[:, n0:n1] has no reduction across column shards, so every rank keeps
the whole compressed A (values + tensor-core metadata), owns a contiguous range of B's and
C's columns and runs the single-GPU kernel on it: no collective is on the data path.  NCCL
is used only when the caller asks for a replicated result; then C is all-gathered, in row
panels so that the gather of one panel overlaps the GEMM of the next.  With replicated="fused"
there is no separate collective at all: every rank's copy of C lives in a buffer that the other
ranks have mapped (`PeerBuffer`), and each rank's GEMM stores its column shard into all copies
from its epilogue, so the shard crosses NVLink tile by tile while the GEMM runs.  With
replicated="copy" the GEMM runs in row panels on its best tile, writing straight into its place in
this rank's copy of C, and each finished panel is pushed to the other ranks' copies by the copy
engines (pitched peer copies on side streams) while the SMs multiply the next panel.

The reference project is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int, multiple: int = 8) -> Tuple[int, int]:
    """[start, end) of rank's column range: `n` split into `world` contiguous ranges whose
    sizes are multiples of `multiple` (the kernel's N granularity) and differ by at most one
    unit; the first ranks get the larger ranges."""
    if n % multiple != 0:
        raise ValueError(f"N={n} must be a multiple of {multiple}")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    units = n // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    size = base + (1 if rank < extra else 0)
    return start * multiple, (start + size) * multiple


def row_panels(m: int, panels: int, multiple: int = 128) -> List[Tuple[int, int]]:
    """split M rows into at most `panels` contiguous panels that start on multiples of `multiple`
    (the row granularity of the tensor-core metadata records); only the last panel may end off one"""
    if m <= 0 or m % 32 != 0:
        raise ValueError(f"M={m} must be a positive multiple of 32")
    units = -(-m // multiple)
    panels = max(1, min(panels, units))
    base, extra = divmod(units, panels)
    out, r = [], 0
    for i in range(panels):
        size = (base + (1 if i < extra else 0)) * multiple
        out.append((r, min(r + size, m)))
        r += size
    return out


class _CudaPeerBackend:
    """exportable device memory through the library's CUDA IPC helpers"""

    def __init__(self, device: torch.device):
        self.device = device

    def alloc(self, nbytes: int) -> int:
        from . import ops
        return ops.peer_alloc(nbytes, self.device)

    def free(self, ptr: int) -> None:
        from . import ops
        ops.peer_free(ptr)

    def export(self, ptr: int) -> bytes:
        from . import ops
        return ops.peer_export(ptr)

    def open(self, handle: bytes) -> int:
        from . import ops
        return ops.peer_open(handle, self.device)

    def close(self, ptr: int) -> None:
        from . import ops
        ops.peer_close(ptr)

    def copy_2d(self, dst: int, dst_pitch: int, src: int, src_pitch: int, width_bytes: int, rows: int, stream) -> None:
        from . import ops
        ops.peer_copy_2d(dst, dst_pitch, src, src_pitch, width_bytes, rows, stream)

    def as_tensor(self, ptr: int, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        class _Raw:   # zero-copy view of the allocation through the CUDA array interface
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (rows * cols,), "typestr": "<i2", "data": (ptr, False),
                                        "strides": None, "version": 3}
        return torch.as_tensor(raw, device=self.device).view(dtype).view(rows, cols)


class PeerBuffer:
    """A (rows, cols) 16-bit matrix per rank, each mapped into every other rank's process.

    `tensor` is this rank's copy; `ptrs[g]` is the address of rank g's copy as seen from this
    rank (its own allocation for g == rank).  Collective over `group`: every rank constructs it
    with the same shape.  `close()` is collective too (mappings are closed everywhere before any
    owner frees).  `backend` supplies alloc / export / open / close / free / as_tensor; the default
    uses CUDA IPC, tests on CPU ranks pass a shared-file stand-in.
    """

    HANDLE_BYTES = 64

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, group=None, backend=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.backend = backend or _CudaPeerBackend(device)
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self._own = self.backend.alloc(rows * cols * 2)
        handle = self.backend.export(self._own)
        if len(handle) != self.HANDLE_BYTES:
            raise RuntimeError(f"peer handle of {len(handle)} bytes, expected {self.HANDLE_BYTES}")
        comm_dev = device if dist.get_backend(group) == "nccl" else torch.device("cpu")
        mine = torch.frombuffer(bytearray(handle), dtype=torch.uint8).to(comm_dev)
        everyone = torch.empty(self.world * self.HANDLE_BYTES, dtype=torch.uint8, device=comm_dev)   # rank-major
        dist.all_gather_into_tensor(everyone, mine, group=group)
        everyone = everyone.cpu().view(self.world, self.HANDLE_BYTES)
        self.ptrs: List[int] = []
        for g in range(self.world):
            self.ptrs.append(self._own if g == self.rank else self.backend.open(bytes(everyone[g].tolist())))
        self.tensor = self.backend.as_tensor(self._own, rows, cols, dtype)
        self._open = True

    def close(self) -> None:
        if not self._open:
            return
        self._open = False
        self.tensor = None
        for g, ptr in enumerate(self.ptrs):
            if g != self.rank:
                self.backend.close(ptr)
        dist.barrier(group=self.group)      # nobody still maps a buffer that is about to be freed
        self.backend.free(self._own)


def _default_scatter(vals, meta_tc, B, dst_ptrs, ldc):
    from . import ops
    ops.spmm_scatter(vals, meta_tc, B, dst_ptrs, ldc)


def _default_spmm(vals, meta_tc, B, out=None):
    from . import ops
    return ops.spmm(vals, meta_tc, B, meta_layout="tc", out=out)


class NShardedSpmm:
    """Sparse GEMM with the output columns sharded over a process group.

    vals / meta_tc : the compressed A, identical on every rank (compress it redundantly on
                     each rank -- a sub-millisecond kernel -- or broadcast it once)
    group          : torch.distributed process group (default: the world group)
    spmm_fn        : the single-device product, `spmm_fn(vals, meta_tc, B_shard, out=...)`;
                     defaults to the tcgen05 kernel.  Tests on CPU ranks pass a stand-in.
    scatter_fn     : the product stored to several destinations (replicated="fused");
                     defaults to `s24_spmm_scatter`.  peer_backend: see `PeerBuffer`.
    """

    def __init__(self, vals: torch.Tensor, meta_tc: torch.Tensor, group=None, spmm_fn: Optional[Callable] = None,
                 scatter_fn: Optional[Callable] = None, peer_backend=None):
        self.vals = vals
        self.meta_tc = meta_tc
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.spmm_fn = spmm_fn or _default_spmm
        self.M = vals.shape[0]
        self.K = vals.shape[1] * 2
        self._comm_stream = None
        self.scatter_fn = scatter_fn or _default_scatter   # scatter_fn(vals, meta_tc, B_shard, dst_ptrs, ldc)
        self.peer_backend = peer_backend
        self._peer: Optional[PeerBuffer] = None
        self._copy_streams: List = []
        self._fence_flag: Optional[torch.Tensor] = None

    def local_columns(self, n_total: int) -> Tuple[int, int]:
        return shard_bounds(n_total, self.world, self.rank)

    def __call__(self, B_shard: torch.Tensor, n_total: Optional[int] = None, replicated=False,
                 panels: int = 4) -> torch.Tensor:
        """B_shard: this rank's (K, N_local) columns of B.  Returns the local (M, N_local)
        shard of C, or with replicated=True the full (M, n_total) C on every rank (all-gather).
        replicated="copy" gives the same result with the shards pushed by the copy engines, panel by
        panel, while the GEMM of the next panel runs (result buffer owned and reused like "fused").
        replicated="auto" picks "copy" on two GPUs and "fused" otherwise.
        replicated="fused" gives the same result without a collective on the data path: the GEMM
        itself stores each shard into every rank's copy of C.  That copy is a buffer owned by this
        object and is returned again (overwritten) by the next fused call of the same shape."""
        if B_shard.shape[0] != self.K:
            raise RuntimeError(f"B shard has {B_shard.shape[0]} rows, expected K={self.K}")
        n_local = B_shard.shape[1]
        if not replicated or self.world == 1:
            return self.spmm_fn(self.vals, self.meta_tc, B_shard)
        if n_total is None:
            n_total = n_local * self.world
        if n_local * self.world != n_total:
            raise RuntimeError("replicated output needs equal column shards on every rank "
                               f"(N_local={n_local}, world={self.world}, N={n_total})")
        if replicated == "auto":
            # measured on cfg 5 (28672 x 8192 x 65536): with two GPUs the GEMM is the longer leg and the
            # copy engines hide the exchange behind it on the GEMM's best tile; from four GPUs on the link
            # is the bound and the fused epilogue, which hides the whole GEMM under it, is faster
            replicated = "copy" if self.world == 2 else "fused"
        if replicated == "fused":
            return self._fused(B_shard, n_total)
        if replicated == "copy":
            return self._copied(B_shard, n_total, panels)
        return self._gathered(B_shard, n_total, panels)

    def _fence(self, device: torch.device) -> None:
        """order the ranks on the current stream without blocking the host: a one-element all-reduce"""
        if self._fence_flag is None or self._fence_flag.device != device:
            self._fence_flag = torch.zeros(1, dtype=torch.int32, device=device)
        dist.all_reduce(self._fence_flag, group=self.group)

    def _fused(self, B_shard: torch.Tensor, n_total: int) -> torch.Tensor:
        M, G, nl = self.M, self.world, B_shard.shape[1]
        dev = B_shard.device
        if self._peer is not None and (self._peer.rows, self._peer.cols) != (M, n_total):
            self._peer.close()
            self._peer = None
        if self._peer is None:
            self._peer = PeerBuffer(M, n_total, self.vals.dtype, dev, group=self.group, backend=self.peer_backend)
        buf = self._peer
        self._fence(dev)          # every rank is done reading the previous result
        col0 = self.rank * nl
        # start with this rank's own copy and go round the ring, so that at any moment the ranks
        # store to different destinations
        order = [(self.rank + i) % G for i in range(G)]
        dsts = [buf.ptrs[g] + 2 * col0 for g in order]
        self.scatter_fn(self.vals, self.meta_tc, B_shard, dsts, n_total)
        self._fence(dev)          # every rank's shard has landed in every copy
        return buf.tensor

    def _copied(self, B_shard: torch.Tensor, n_total: int, panels: int) -> torch.Tensor:
        M, G, nl = self.M, self.world, B_shard.shape[1]
        dev = B_shard.device
        if self._peer is not None and (self._peer.rows, self._peer.cols) != (M, n_total):
            self._peer.close()
            self._peer = None
        if self._peer is None:
            self._peer = PeerBuffer(M, n_total, self.vals.dtype, dev, group=self.group, backend=self.peer_backend)
        buf = self._peer
        cuda = dev.type == "cuda"
        if cuda and not self._copy_streams:
            self._copy_streams = [torch.cuda.Stream(device=dev) for _ in range(G - 1)]   # one per destination
        compute = torch.cuda.current_stream(dev) if cuda else None
        self._fence(dev)          # every rank is done reading the previous result
        col0 = self.rank * nl
        pitch = n_total * 2
        mine = buf.tensor[:, col0:col0 + nl]               # this rank's columns of its own copy
        for (r0, r1) in row_panels(M, panels):
            # the panel's product lands in place: row stride n_total, no staging buffer
            self.spmm_fn(self.vals[r0:r1], self._meta_rows(r0, r1), B_shard, out=mine[r0:r1])
            off = (r0 * n_total + col0) * 2
            ev = None
            if cuda:
                ev = torch.cuda.Event()
                ev.record(compute)
            # round the ring starting after this rank, so that at any moment the ranks push to different peers
            for i in range(1, G):
                g = (self.rank + i) % G
                st = self._copy_streams[i - 1] if cuda else None
                if cuda:
                    st.wait_event(ev)
                self.backend_copy(buf, buf.ptrs[g] + off, pitch, buf.ptrs[self.rank] + off, pitch, nl * 2, r1 - r0, st)
        if cuda:
            for st in self._copy_streams:
                done = torch.cuda.Event()
                done.record(st)
                compute.wait_event(done)
        self._fence(dev)          # every rank's panels have landed in every copy
        return buf.tensor

    @staticmethod
    def backend_copy(buf: "PeerBuffer", dst, dst_pitch, src, src_pitch, width_bytes, rows, stream) -> None:
        buf.backend.copy_2d(dst, dst_pitch, src, src_pitch, width_bytes, rows, stream)

    def close(self) -> None:
        """release the peer-mapped result buffer (collective)"""
        if self._peer is not None:
            self._peer.close()
            self._peer = None

    def _gathered(self, B_shard: torch.Tensor, n_total: int, panels: int) -> torch.Tensor:
        M, G, nl = self.M, self.world, B_shard.shape[1]
        dev = B_shard.device
        out = torch.empty((M, n_total), dtype=self.vals.dtype, device=dev)
        out_v = out.view(M, G, nl)
        cuda = dev.type == "cuda"
        if cuda and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=dev)
        compute = torch.cuda.current_stream(dev) if cuda else None
        pending = []
        for (r0, r1) in row_panels(M, panels):
            rows = r1 - r0
            c_local = self.spmm_fn(self.vals[r0:r1], self._meta_rows(r0, r1), B_shard)
            stage = torch.empty((G * rows, nl), dtype=c_local.dtype, device=dev)   # rank-major concatenation
            if cuda:
                ev = torch.cuda.Event()
                ev.record(compute)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ev)
                    dist.all_gather_into_tensor(stage, c_local.contiguous(), group=self.group)
                    self._relayout(stage.view(G, rows, nl), out[r0:r1])             # shard-major -> row-major
                    done = torch.cuda.Event()
                    done.record(self._comm_stream)
                pending.append((done, stage, c_local))
            else:
                dist.all_gather_into_tensor(stage, c_local.contiguous(), group=self.group)
                out_v[r0:r1].copy_(stage.view(G, rows, nl).permute(1, 0, 2))
        if cuda:
            for done, _, _ in pending:
                compute.wait_event(done)
        return out

    @staticmethod
    def _relayout(stage3: torch.Tensor, out_rows: torch.Tensor) -> None:
        if stage3.is_cuda and stage3.element_size() == 2 and stage3.shape[2] % 8 == 0:
            from . import ops
            ops.relayout_shards(stage3, out_rows)          # the library's copy kernel
        else:                                              # CPU ranks in tests
            G, rows, nl = stage3.shape
            out_rows.view(rows, G, nl).copy_(stage3.permute(1, 0, 2))

    def _meta_rows(self, r0: int, r1: int) -> torch.Tensor:
        """tensor-core metadata of rows [r0, r1): records are ordered [row tile of 128][k block],
        512 int32 each, so a row panel is a contiguous slice"""
        per_tile = -(-self.K // 128) * 512
        return self.meta_tc[(r0 // 128) * per_tile:-(-r1 // 128) * per_tile]
