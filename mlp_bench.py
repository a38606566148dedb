"""Multi-GPU MLP-shaped sparse GEMM: 2:4-sparse bf16 weight W (28672 x 8192, ~N(0, 0.02)) times
activations X (8192 x 65536, ~N(0, 1)), output columns sharded over the ranks (strong scaling:
the 65536 columns are split over 1 / 2 / 4 / 8 GPUs), without a replicated result, with one made
by an NCCL all-gather, and with one made by the GEMM storing each shard into all ranks' copies.  Launch one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
        mlp_bench.py [--steps 10]

Rank 0 prints one JSON line: aggregate dense-equivalent TFLOP/s (max-over-ranks device time)
for the sharded result and for the two replicated ones.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent / "gpu-compression-kernel_b200"))
import s24  # noqa: E402
from s24.multi import NShardedSpmm  # noqa: E402

M, K, N = 28672, 8192, 65536


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--gather-steps", type=int, default=3)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    g = torch.Generator(device=dev).manual_seed(5000)                    # same W on every rank
    W = (0.02 * torch.randn(M, K, generator=g, device=dev, dtype=torch.float32)).to(torch.bfloat16)
    vals, _, tc = s24.prune_compress(W, want_ref=False, want_tc=True)    # compressed redundantly, no broadcast
    del W
    op = NShardedSpmm(vals, tc)
    n0, n1 = op.local_columns(N)
    gx = torch.Generator(device=dev).manual_seed(5001 + rank)
    X = torch.randn(K, n1 - n0, generator=gx, device=dev, dtype=torch.float32).to(torch.bfloat16)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        for _ in range(2):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        b.synchronize()
        t = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        barrier()
        return float(t.item())

    flops = 2.0 * M * N * K
    ms_shard = timed(lambda: op(X), args.steps)
    line = {"workload": f"W24 {M}x{K} bf16 . X {K}x{N} bf16, columns sharded x{world}", "n_gpus": world,
            "sharded": {"ms": ms_shard, "tflops": flops / ms_shard / 1e9}}
    if world > 1:
        ms_rep = timed(lambda: op(X, n_total=N, replicated=True, panels=8), args.gather_steps)
        line["replicated"] = {"ms": ms_rep, "tflops": flops / ms_rep / 1e9,
                              "gathered_bytes_per_gpu": M * N * 2 * (world - 1) // world}
        # the same replicated result with the shard stored into every rank's copy of C by the GEMM's
        # own epilogue (peer-mapped buffers, no collective on the data path)
        ms_fused = timed(lambda: op(X, n_total=N, replicated="fused"), args.gather_steps)
        line["replicated_fused"] = {"ms": ms_fused, "tflops": flops / ms_fused / 1e9,
                                    "stored_to_peers_bytes_per_gpu": M * (N // world) * 2 * (world - 1)}
        op.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
