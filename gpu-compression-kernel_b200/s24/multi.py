"""N-sharded sparse GEMM across the GPUs of one box (one process per GPU).

C[:, n0:n1] = A24 . B[:, n0:n1] has no reduction across column shards, so every rank keeps
the whole compressed A (values + tensor-core metadata), owns a contiguous range of B's and
C's columns and runs the single-GPU kernel on it: no collective is on the data path.  NCCL
is used only when the caller asks for a replicated result; then C is all-gathered, in row
panels so that the gather of one panel overlaps the GEMM of the next.

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
    """split M rows into at most `panels` contiguous panels whose sizes are multiples of
    `multiple` (the kernel's M granularity)"""
    if m % multiple != 0:
        raise ValueError(f"M={m} must be a multiple of {multiple}")
    units = m // multiple
    panels = max(1, min(panels, units))
    base, extra = divmod(units, panels)
    out, r = [], 0
    for i in range(panels):
        size = (base + (1 if i < extra else 0)) * multiple
        out.append((r, r + size))
        r += size
    return out


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
    """

    def __init__(self, vals: torch.Tensor, meta_tc: torch.Tensor, group=None, spmm_fn: Optional[Callable] = None):
        self.vals = vals
        self.meta_tc = meta_tc
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.spmm_fn = spmm_fn or _default_spmm
        self.M = vals.shape[0]
        self.K = vals.shape[1] * 2
        self._comm_stream = None

    def local_columns(self, n_total: int) -> Tuple[int, int]:
        return shard_bounds(n_total, self.world, self.rank)

    def __call__(self, B_shard: torch.Tensor, n_total: Optional[int] = None, replicated: bool = False,
                 panels: int = 4) -> torch.Tensor:
        """B_shard: this rank's (K, N_local) columns of B.  Returns the local (M, N_local)
        shard of C, or with replicated=True the full (M, n_total) C on every rank."""
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
        return self._gathered(B_shard, n_total, panels)

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
        per_tile = (self.K // 128) * 512
        return self.meta_tc[(r0 // 128) * per_tile:(r1 // 128) * per_tile]
