"""N-sharded sparse GEMM on two GPUs (one process per GPU, NCCL): local shards, the all-gathered
replicated result and the one stored into peer-mapped buffers by the GEMM itself, against a
single-GPU product.  Skipped on a one-GPU box."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

RANK_SCRIPT = r'''
import os, sys
sys.path.insert(0, "{root}"); sys.path.insert(0, "{root}/gpu-compression-kernel_b200")
import torch, torch.distributed as dist
import s24
from s24.multi import NShardedSpmm
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
import datetime
dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
torch.backends.cuda.matmul.allow_tf32 = False
M, K, N = 1024, 1024, 512 * world
g = torch.Generator().manual_seed(99)
A = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
B = torch.randn(K, N, generator=g).to(torch.bfloat16).to(dev)
vals, _, tc = s24.prune_compress(A, want_ref=False, want_tc=True)      # redundantly on every rank
op = NShardedSpmm(vals, tc)
n0, n1 = op.local_columns(N)
C_local = op(B[:, n0:n1].contiguous())
ref = s24.prune(A).float() @ B.float()
torch.testing.assert_close(C_local.float(), ref[:, n0:n1], rtol=1e-2, atol=1e-2 + 8e-3 * float(ref.abs().max()))
C_full = op(B[:, n0:n1].contiguous(), n_total=N, replicated=True, panels=4)
torch.cuda.synchronize()
torch.testing.assert_close(C_full.float(), ref, rtol=1e-2, atol=1e-2 + 8e-3 * float(ref.abs().max()))
single = s24.spmm(vals, tc, B)
assert torch.equal(C_full, single), "gathered result differs from the single-GPU product"
# replicated result without a collective on the data path: each rank's GEMM stores its shard into
# every rank's peer-mapped copy of C; bit-identical to the single-GPU product on the same tile
want = s24.spmm(vals, tc, B, manual_config={{"BM": 256, "BN": 256}})
for it in range(3):
    Bi = B if it == 0 else torch.roll(B, it, dims=0)
    wi = want if it == 0 else s24.spmm(vals, tc, Bi, manual_config={{"BM": 256, "BN": 256}})
    C_fused = op(Bi[:, n0:n1].contiguous(), n_total=N, replicated="fused")
    torch.cuda.synchronize()
    assert torch.equal(C_fused, wi), f"fused replicated result differs (iteration {{it}})"
# the same replicated result with the shards pushed by the copy engines, row panel by row panel, while
# the next panel multiplies; the GEMM writes in place with its default tiles
for it in range(3):
    Bi = B if it == 0 else torch.roll(B, it, dims=0)
    wi = single if it == 0 else s24.spmm(vals, tc, Bi)
    C_copy = op(Bi[:, n0:n1].contiguous(), n_total=N, replicated="copy", panels=4)
    torch.cuda.synchronize()
    assert torch.equal(C_copy, wi), f"copy-engine replicated result differs (iteration {{it}})"
from s24 import _lib
assert _lib.lib().s24_device_status(None) == 0, _lib.last_error()
op.close()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_nshard(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT.format(root=str(ROOT)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("ok") == 2
