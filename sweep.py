"""Shape sweep of the 2:4 path, the counterpart of the reference's benchmark drivers
(compression/dev/8.11_benchmark_2_kernel.py:205-265 for the GEMM lines,
compression/dev/8.11.1_benchmark_pruning.py for prune+compress,
compression/dev/8.10_benchmark_post_compression.py for the fused-output lines).

    python sweep.py [--n 8192] [--dtype fp16|bf16] [--quick] [--out results.jsonl]
    python sweep.py --table results.jsonl        # markdown table, no GPU needed

For every (M, K) of the reference's 13 x 13 grid (N fixed) it appends one JSON line with, in
the reference's units (dense-equivalent TFLOP/s = 2 M N K / t, GB/s = 3.125 M K / t):

  dense        torch.matmul of the pruned dense A (cuBLAS; stands in for the reference's dense WS kernel)
  sparse       precompressed sparse GEMM (gluon_ws_sparse.py: run_sparse_ws_matmul)
  two_kernel   prune+compress kernel then sparse GEMM (v11.1: run_2_kernel_ws_matmul)
  fused_in     sparse GEMM that prunes + compresses the dense A inside the kernel (v7.8.1)
  fused_out    sparse GEMM with the pruning epilogue (v10.1)
  separated    sparse GEMM then prune+compress of C (v10.2)
  compress     the standalone prune+compress kernel, GB/s

Shapes are visited largest first like the reference does (8.11_benchmark_2_kernel.py:244);
lines are appended as they are measured, so an interrupted sweep can be resumed with --skip-done.
Inputs are seeded randn (the reference uses unseeded randn).  Timing: CUDA events around enough
back-to-back launches to fill about 30 ms, after 3 warm-ups.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "gpu-compression-kernel_b200"))
import s24  # noqa: E402

GRID = [768, 1024, 1536, 2048, 3072, 4096, 6144, 8192, 12288, 16384, 24576, 32768, 49152]
QUICK = [2048, 4096, 8192, 16384]


USE_GRAPH = True


def timeit(fn, target_ms=30.0):
    """ms per call.  Like the reference's triton.testing.do_bench_cudagraph
    (dev/8.11_benchmark_2_kernel.py:52-61) the calls are captured into one CUDA graph and the
    replay is timed, so host-side launch cost does not count; --eager times plain launches."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    b.synchronize()
    one = max(a.elapsed_time(b), 1e-3)
    n = int(max(3, min(200, target_ms / one)))
    if USE_GRAPH:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(n):
                    fn()
            g.replay()
            torch.cuda.synchronize()
            a.record()
            g.replay()
            b.record()
            b.synchronize()
            ms = a.elapsed_time(b) / n
            del g
            return ms
        except Exception:
            torch.cuda.synchronize()
    a.record()
    for _ in range(n):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / n


def print_table(path: str) -> int:
    """render a results file of this script as a markdown table (no GPU needed)"""
    recs = {}
    for line in Path(path).read_text().splitlines():
        try:
            d = json.loads(line)
            recs[(d["M"], d["K"])] = d          # a re-measured shape replaces its earlier line
        except Exception:
            continue
    if not recs:
        print(f"no records in {path}", file=sys.stderr)
        return 1
    cols = [c for c in ("dense", "sparse", "sparse_untuned", "sparse_ref_meta", "two_kernel", "fused_in", "fused_out", "separated",
                        "vendor_sparse", "vendor_two_step", "compress_gbs") if any(c in d for d in recs.values())]
    print("| M | K | " + " | ".join(cols) + " |")
    print("|---|---|" + "---|" * len(cols))
    for (m, k) in sorted(recs, key=lambda mk: (-mk[0] * mk[1], -mk[0])):
        d = recs[(m, k)]
        print(f"| {m} | {k} | " + " | ".join(f"{d[c]:.0f}" if c in d else "-" for c in cols) + " |")
    lose = [(m, k) for (m, k), d in recs.items() if "sparse" in d and "dense" in d and d["sparse"] < d["dense"]]
    means = {c: sum(d[c] for d in recs.values() if c in d) / max(1, sum(1 for d in recs.values() if c in d)) for c in cols}
    print("| mean | | " + " | ".join(f"{means[c]:.0f}" for c in cols) + " |")
    print(f"\nsparse below dense on {len(lose)} of {len(recs)} shapes: {sorted(lose)}")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--dtype", choices=["fp16", "bf16"], default="fp16")
    ap.add_argument("--quick", action="store_true", help="4 x 4 grid instead of 13 x 13")
    ap.add_argument("--out", default="-")
    ap.add_argument("--skip-done", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time plain launches instead of CUDA-graph replays")
    ap.add_argument("--vendor", action="store_true",
                    help="also time torch's semi-structured sparse matmul (cuSPARSELt / CUTLASS behind "
                         "torch.sparse.to_sparse_semi_structured), the stand-in for the reference's torchao line")
    ap.add_argument("--max-elems", type=float, default=2.5e9, help="skip shapes whose M*K exceeds this")
    ap.add_argument("--table", metavar="RESULTS.jsonl", default=None,
                    help="print a results file as a markdown table (TFLOP/s; last column GB/s) and exit")
    args = ap.parse_args()
    if args.table:
        return print_table(args.table)
    global USE_GRAPH
    USE_GRAPH = not args.eager
    dtype = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    dev = torch.device("cuda", 0)
    N = args.n
    grid = QUICK if args.quick else GRID
    shapes = sorted(((m, k) for m in grid for k in grid), key=lambda mk: -mk[0] * mk[1])
    done = set()
    out = sys.stdout
    if args.out != "-":
        p = Path(args.out)
        if args.skip_done and p.exists():
            for line in p.read_text().splitlines():
                try:
                    d = json.loads(line)
                    done.add((d["M"], d["K"]))
                except Exception:
                    pass
        out = open(p, "a")
    for idx, (M, K) in enumerate(shapes):
        if (M, K) in done or M * K > args.max_elems:
            continue
        g = torch.Generator(device=dev).manual_seed(3000 + idx)
        A = torch.randn(M, K, generator=g, device=dev, dtype=torch.float32).to(dtype)
        B = torch.randn(K, N, generator=g, device=dev, dtype=torch.float32).to(dtype)
        A_pruned = s24.prune(A)
        vals, E, tc = s24.prune_compress(A, want_ref=True, want_tc=True)
        C = torch.empty(M, N, dtype=dtype, device=dev)
        flops = 2.0 * M * N * K
        rec = {"M": M, "N": N, "K": K, "dtype": args.dtype}
        # the bandwidth-bound kernel first, after a short pause: right after a run of GEMMs the
        # board is still at its power-capped clock, which would be charged to this kernel
        torch.cuda.synchronize()
        time.sleep(0.05)
        ms = timeit(lambda: s24.prune_compress(A, want_ref=True, want_tc=False))
        rec["compress_gbs"] = round(3.125 * M * K / ms / 1e6, 1)
        rec["compress_ms"] = round(ms, 4)

        def tf(ms):
            return round(flops / ms / 1e9, 1)

        rec["dense"] = tf(timeit(lambda: torch.matmul(A_pruned, B, out=C)))
        # like the reference's launchers (tune=True, gluon_ws_sparse.py:572-582) the GEMM lines run the tile
        # shape an autotune pass picked for this (M, N, K); the library's untuned heuristic is timed beside it
        from s24.ops import _autotune
        tuned = _autotune(vals, tc, B, C, M, N, K)
        rec["tile"] = "heuristic" if tuned is None else f"{tuned['BM']}x{tuned['BN']}"
        rec["sparse"] = tf(timeit(lambda: s24.spmm(vals, tc, B, out=C, manual_config=tuned)))
        rec["sparse_untuned"] = tf(timeit(lambda: s24.spmm(vals, tc, B, out=C)))
        rec["sparse_ref_meta"] = tf(timeit(lambda: s24.spmm(vals, E, B, meta_layout="ref", out=C, manual_config=tuned)))

        def two_kernel():
            v, _, t = s24.prune_compress(A, tie="higher", want_ref=False, want_tc=True)
            s24.spmm(v, t, B, out=C, manual_config=tuned)

        rec["two_kernel"] = tf(timeit(two_kernel))
        rec["fused_in"] = tf(timeit(lambda: s24.spmm_prune_in(A, B, out=C)))
        if args.vendor:
            try:
                from torch.sparse import to_sparse_semi_structured
                A_sp = to_sparse_semi_structured(A_pruned)
                rec["vendor_sparse"] = tf(timeit(lambda: torch.mm(A_sp, B)))

                def vendor_e2e():
                    torch.mm(to_sparse_semi_structured(s24.prune(A)), B)

                rec["vendor_two_step"] = tf(timeit(vendor_e2e))
                del A_sp
            except Exception as exc:  # library missing or shape unsupported on this box
                rec["vendor_error"] = f"{type(exc).__name__}: {exc}"[:200]
        if N % 128 == 0:
            rec["fused_out"] = tf(timeit(lambda: s24.spmm_prune_out(vals, tc, B)))

            def separated():
                s24.spmm(vals, tc, B, out=C)
                s24.prune_compress(C, tie="higher")

            rec["separated"] = tf(timeit(separated))
        out.write(json.dumps(rec) + "\n")
        out.flush()
        del A, B, A_pruned, vals, E, tc, C
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
