"""torch-tensor front end of the C ABI.

Each function validates its tensors the way the reference's functions do (same
exception types for the same conditions), allocates outputs with torch on the input's
device (so the caller's allocator and CUDA-graph capture work as with the reference,
gluon_ws_sparse.py:563), and enqueues the library call on torch's current stream.
There is no fallback: CPU tensors or a missing libs24.so raise.
"""
from __future__ import annotations

import ctypes
import os
import sys
from typing import Optional, Tuple

import torch

from . import _lib as L

_DT = {torch.float16: L.FP16, torch.bfloat16: L.BF16}
_MODE = {"signed": L.MODE_SIGNED, "magnitude": L.MODE_MAGNITUDE}
_TIE = {"reference": L.TIE_REFERENCE, "torch": L.TIE_REFERENCE, "lower": L.TIE_LOWER, "higher": L.TIE_HIGHER}


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


# S24_NVTX=1 wraps every library call in an NVTX range named after the calling front-end function,
# the way the reference brackets its launches for Nsight (compression/dev/9.4_profile_ws.py:48-53)
_NVTX = os.environ.get("S24_NVTX", "0") not in ("", "0")


class _on_device:
    """`with _on_device(t):` makes t's device current for the library call; a no-op (and much
    cheaper than torch.cuda.device) when it already is, which is the common case"""
    __slots__ = ("idx", "prev", "ranged")

    def __init__(self, t: torch.Tensor):
        self.idx = t.device.index
        self.prev = None
        self.ranged = False

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        if _NVTX:
            torch.cuda.nvtx.range_push("s24." + sys._getframe(1).f_code.co_name)
            self.ranged = True

    def __exit__(self, *exc):
        if self.ranged:
            torch.cuda.nvtx.range_pop()
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


# S24_CHECK_STATUS=1: after every GEMM call synchronise the stream and raise if a bounded
# device-side wait gave up (the launch itself reports success and leaves C partly written in that
# case).  Off by default because it serialises host and device; callers that keep it off should
# poll s24_device_status at their own synchronisation points.
_CHECK_STATUS = os.environ.get("S24_CHECK_STATUS", "0") not in ("", "0")


def _after_gemm(t: torch.Tensor) -> None:
    if _CHECK_STATUS and not torch.cuda.is_current_stream_capturing():
        L.check(L.lib().s24_device_status(_stream(t)))


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("s24 kernels run on CUDA tensors only (there is no CPU path)")
    dev = {t.device for t in ts if t is not None}
    if len(dev) > 1:
        raise RuntimeError(f"tensors live on different devices: {sorted(map(str, dev))}")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise RuntimeError(f"Invalid datatype {t.dtype} of dense matrix")
    return _DT[t.dtype]


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def meta_tc_numel(M: int, K: int) -> int:
    """int32 elements of a tensor-core-layout metadata buffer for an (M, K) matrix."""
    return int(L.lib().s24_meta_tc_bytes(M, K)) // 4


def _new_meta_tc(M: int, K: int, device) -> torch.Tensor:
    """Tensor-core-layout buffer.  Records are whole (128-row tile, 128-column block) units; when the
    matrix covers the last ones only partly, the library call that fills the buffer also gives the
    words outside the matrix a valid code (the values they index are zero)."""
    return torch.empty((meta_tc_numel(M, K),), dtype=torch.int32, device=device)


def prune(t: torch.Tensor, mode: str = "signed", tie: str = "reference") -> torch.Tensor:
    """2:4 prune along the last dimension; new tensor (compression/prune.py:57-96)."""
    if t.size(-1) % 4 != 0:
        raise ValueError("The size of the last dimension must be divisible by 4.")
    _require_cuda(t)
    dt = _dtype_code(t)
    src = t.contiguous()
    out = torch.empty_like(src)
    with _on_device(t):
        L.check(L.lib().s24_prune(_p(src), _p(out), src.numel(), dt, _MODE[mode], _TIE[tie], _stream(t)))
    return out.view(t.shape)


def _check_compress_shape(dense: torch.Tensor) -> Tuple[int, int]:
    # same conditions and exception types as compress_2_4.py:33-65 and :10
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    _dtype_code(dense)
    m, k = dense.shape
    if m % 32 != 0:
        raise RuntimeError(f"Number of rows of dense matrix {m} must be divisible by 32")
    if k % 16 != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by 16")
    assert (k // 16) % 4 == 0, f"The number of metadata cols must be at least 4, current number: {k // 16}"
    return m, k


def _row_major(t: torch.Tensor) -> torch.Tensor:
    if t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.stride(0) < t.shape[1] or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


def compress(dense: torch.Tensor, want_ref: bool = True, want_tc: bool = False):
    """compress_dense_to_sparse from non-zero flags (compression/compress_2_4.py:32-161).

    Returns (values (M, K/2), E (M/16, K) int16 or None, meta_tc int32 or None).
    """
    m, k = _check_compress_shape(dense)
    _require_cuda(dense)
    d = _row_major(dense)
    vals = torch.empty((m, k // 2), dtype=dense.dtype, device=dense.device)
    e = torch.empty((m // 16, k), dtype=torch.int16, device=dense.device) if want_ref else None
    tc = _new_meta_tc(m, k, dense.device) if want_tc else None
    if m * k:
        with _on_device(dense):
            L.check(L.lib().s24_compress(_p(d), m, k, d.stride(0), _DT[dense.dtype], _p(vals), _p(e), _p(tc),
                                         _stream(dense)))
    return vals, e, tc


_OTHER = {torch.int8: (L.INT8, torch.int32, 16, 8, 4), torch.int32: (L.INT32, torch.int16, 32, 4, 4),
          torch.float32: (L.FP32, torch.int16, 32, 4, 2)}   # code, metadata type, row multiple, codes per word, group size


def compress_other(dense: torch.Tensor):
    """compress_dense_to_sparse for int8 / int32 / float32 input (compression/compress_2_4.py:41-47,73-76,
    144-154): returns (values (M, K/2), reordered metadata viewed (M/2, 2 * words per row)), with the
    reference's exception types for the shapes it rejects."""
    if dense.dim() != 2:
        raise RuntimeError(f"Expected 2-dimensional dense tensor, got {dense.dim()}-dimensional tensor")
    if dense.dtype not in _OTHER:
        raise RuntimeError(f"Invalid datatype {dense.dtype} of dense matrix")
    code, meta_dtype, row_mult, codes, ksparse = _OTHER[dense.dtype]
    m, k = dense.shape
    if m % row_mult != 0:
        raise RuntimeError(f"Number of rows of dense matrix {m} must be divisible by {row_mult}")
    if k % (4 * codes) != 0:
        raise RuntimeError(f"Number of columns of dense matrix {k} must be divisible by {4 * codes}")
    if m * k == 0:
        return dense, torch.zeros(dense.shape, dtype=meta_dtype, device=dense.device)
    ncols = k // (ksparse * codes)
    assert ncols % 4 == 0, f"The number of metadata cols must be at least 4, current number: {ncols}"
    _require_cuda(dense)
    d = dense
    if d.stride(1) != 1 or (d.stride(0) * d.element_size()) % 16 != 0 or d.stride(0) < k or d.data_ptr() % 16 != 0:
        d = d.contiguous()
    vals = torch.empty((m, k // 2), dtype=dense.dtype, device=dense.device)
    meta = torch.empty((m * ncols,), dtype=meta_dtype, device=dense.device)
    with _on_device(dense):
        L.check(L.lib().s24_compress_other(_p(d), m, k, d.stride(0), code, _p(vals), _p(meta), _stream(dense)))
    return vals, meta.view(-1, 2 * ncols)


def prune_compress(A: torch.Tensor, mode: str = "signed", tie: str = "reference", want_ref: bool = True,
                   want_tc: bool = False):
    """Fused prune + compress, one pass over A (kernels/11.1_2_kernel_baseline.py:171-203,256-279).

    Returns (values (M, K/2), E (M/16, K) int16 or None, meta_tc int32 or None).
    """
    m, k = _check_compress_shape(A)
    _require_cuda(A)
    a = _row_major(A)
    vals = torch.empty((m, k // 2), dtype=A.dtype, device=A.device)
    e = torch.empty((m // 16, k), dtype=torch.int16, device=A.device) if want_ref else None
    tc = _new_meta_tc(m, k, A.device) if want_tc else None
    if m * k:
        with _on_device(A):
            L.check(L.lib().s24_prune_compress(_p(a), m, k, a.stride(0), _DT[A.dtype], _MODE[mode], _TIE[tie],
                                               _p(vals), _p(e), _p(tc), _stream(A)))
    return vals, e, tc


_LAYOUT = {"logical": L.META_LOGICAL, "ref": L.META_REF, "tc": L.META_TC}


def meta_convert(src: torch.Tensor, from_layout: str, to_layout: str, M: int, K: int) -> torch.Tensor:
    """Re-lay metadata of an (M, K) matrix between "logical", "ref" and "tc"."""
    _require_cuda(src)
    src = src.contiguous()
    if to_layout == "tc":
        dst = _new_meta_tc(M, K, src.device)
    elif to_layout == "ref":
        dst = torch.empty((M // 16, K), dtype=torch.int16, device=src.device)
    else:
        dst = torch.empty((M, K // 16), dtype=torch.int16, device=src.device)
    with _on_device(src):
        L.check(L.lib().s24_meta_convert(_p(src), _LAYOUT[from_layout], _p(dst), _LAYOUT[to_layout], M, K,
                                         _stream(src)))
    return dst


def _tile_cfg(manual_config: Optional[dict]):
    if not manual_config:
        return None
    # the ring depth ("buffers" in the reference's configs) is fixed per tile shape here
    cfg = L.TileCfg(int(manual_config.get("BM", 0)), int(manual_config.get("BN", 0)), 0, 0)
    return ctypes.byref(cfg)


def _check_gemm(vals: torch.Tensor, B: torch.Tensor) -> Tuple[int, int, int]:
    if vals.dim() != 2 or B.dim() != 2:
        raise RuntimeError("sparse matmul expects 2-dimensional operands")
    M, K2 = vals.shape
    K, N = B.shape
    if 2 * K2 != K:
        raise RuntimeError(f"compressed A has {K2} columns but B has {K} rows (expected K/2 = {K // 2})")
    if vals.dtype != B.dtype:
        raise RuntimeError(f"operand dtypes differ: {vals.dtype} vs {B.dtype}")
    _dtype_code(vals)
    if M % 32 != 0 or K % 64 != 0 or N % 8 != 0:
        raise RuntimeError(f"sparse matmul needs M % 32 == 0, K % 64 == 0, N % 8 == 0 (got M={M}, N={N}, K={K})")
    return M, N, K


def _check_meta_tc(meta: torch.Tensor, M: int, K: int) -> None:
    """the kernel reads whole records: a short buffer would be read past its end"""
    need = meta_tc_numel(M, K) * 4
    have = meta.numel() * meta.element_size()
    if have < need or not meta.is_contiguous():
        raise RuntimeError(f"tensor-core metadata of a ({M}, {K}) matrix needs {need} contiguous bytes, got {have}")


_TILE_CANDIDATES = ({"BM": 512, "BN": 224}, {"BM": 256, "BN": 256}, {"BM": 256, "BN": 128}, {"BM": 128, "BN": 128})
_TUNED = {}   # (M, N, K, dtype, device index) -> tile config chosen by timing


def _autotune(vals, meta_tc, b, c, M, N, K):
    """Time every tile shape once for this problem (CUDA events, about a millisecond of launches each) and
    remember the fastest, like the reference's Triton autotuner keyed on (M, N, K)
    (compression/gluon_ws_sparse.py:528-535).  Synchronises, so it is skipped during stream capture."""
    key = (M, N, K, vals.dtype, vals.device.index)
    if key in _TUNED:
        return _TUNED[key]
    if torch.cuda.is_current_stream_capturing():
        return None
    stream = torch.cuda.current_stream(vals.device)
    timings = {}
    # None = the library's own heuristic; a named tile must beat it by 3 % to replace it, so that
    # timing noise cannot select a clearly worse shape
    for cfg in (None,) + _TILE_CANDIDATES:
        tc = _tile_cfg(cfg)

        def launch():
            L.check(L.lib().s24_spmm(_p(vals), _p(meta_tc), _p(b), _p(c), M, N, K, b.stride(0), c.stride(0),
                                     _DT[vals.dtype], tc, _stream(vals)))
        launch()
        launch()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        launch()
        e1.record(stream)
        e1.synchronize()
        # About a millisecond of launches, replayed from a CUDA graph so that the host's launch cost
        # (larger than the kernel itself for microsecond-sized problems) does not hide the difference
        # between tile shapes; plain launches if the capture is refused.
        n = int(max(5, min(50, 1.0 / max(e0.elapsed_time(e1), 1e-3))))
        graph = None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(n):
                    launch()
            graph.replay()
        except Exception:
            graph = None
            torch.cuda.synchronize(vals.device)
        best_of = []
        for _ in range(2):
            e0.record(stream)
            if graph is not None:
                graph.replay()
            else:
                for _ in range(n):
                    launch()
            e1.record(stream)
            e1.synchronize()
            best_of.append(e0.elapsed_time(e1) / n)
        del graph
        timings[None if cfg is None else (cfg["BM"], cfg["BN"])] = min(best_of)
    best, best_ms = None, timings[None]
    for cfg in _TILE_CANDIDATES:
        ms = timings[(cfg["BM"], cfg["BN"])]
        if ms < 0.97 * best_ms:
            best, best_ms = cfg, ms
    _TUNED[key] = best
    return best


def spmm(vals: torch.Tensor, meta: torch.Tensor, B: torch.Tensor, meta_layout: str = "tc",
         manual_config: Optional[dict] = None, out: Optional[torch.Tensor] = None,
         workspace: Optional[torch.Tensor] = None, autotune: bool = False) -> torch.Tensor:
    """C = A24 @ B with fp32 accumulation (compression/gluon_ws_sparse.py:560-613).

    meta_layout "tc": `meta` is the tensor-core layout.  "ref": `meta` is the reference's
    E (M/16, K) int16; it is re-laid into `workspace` (allocated here if not given) first.

    B is (K, N).  If it is the transposed view of a row-major (N, K) tensor (`X.t()` of
    activations stored (tokens, hidden)) it is used in place through `s24_spmm_bt`; any other
    non-row-major B is copied to row-major first.
    """
    _require_cuda(vals, meta, B)
    M, N, K = _check_gemm(vals, B)
    v = vals.contiguous()
    bt = (B.stride(0) == 1 and B.stride(1) >= K and B.stride(1) % 8 == 0 and B.data_ptr() % 16 == 0
          and not (B.stride(1) == 1 and B.stride(0) >= N))
    if bt:
        if meta_layout == "ref":
            if meta.numel() != M * K // 16:
                raise RuntimeError(f"E has {meta.numel()} elements, expected {M * K // 16} for ({M}, {K})")
            meta = meta_convert(meta, "ref", "tc", M, K)
        c = out if out is not None else torch.empty((M, N), dtype=vals.dtype, device=vals.device)
        if c.stride(1) != 1 or c.stride(0) % 8 != 0 or tuple(c.shape) != (M, N) or c.dtype != vals.dtype:
            raise RuntimeError(f"`out` must be a row-major ({M}, {N}) {vals.dtype} tensor")
        with _on_device(vals):
            _check_meta_tc(meta, M, K)
            L.check(L.lib().s24_spmm_bt(_p(v), _p(meta), _p(B), _p(c), M, N, K, B.stride(1), c.stride(0),
                                        _DT[vals.dtype], _tile_cfg(manual_config), _stream(vals)))
            _after_gemm(vals)
        return c
    b = _row_major(B)
    if out is not None:
        if (tuple(out.shape) != (M, N) or out.dtype != vals.dtype or out.device != vals.device or out.stride(1) != 1
                or out.stride(0) % 8 != 0 or out.data_ptr() % 16 != 0):
            raise RuntimeError(f"`out` must be a ({M}, {N}) {vals.dtype} tensor on {vals.device} with unit column "
                               "stride, a row stride that is a multiple of 8 and 16-byte alignment")
    c = out if out is not None else torch.empty((M, N), dtype=vals.dtype, device=vals.device)
    with _on_device(vals):
        if meta_layout == "ref" and autotune and manual_config is None:
            # tune on the converted metadata, then run through the native-layout entry point
            if meta.numel() != M * K // 16:
                raise RuntimeError(f"E has {meta.numel()} elements, expected {M * K // 16} for ({M}, {K})")
            meta = meta_convert(meta, "ref", "tc", M, K)
            meta_layout = "tc"
        if autotune and manual_config is None and meta_layout == "tc":
            manual_config = _autotune(v, meta, b, c, M, N, K)
        cfg = _tile_cfg(manual_config)
        if meta_layout == "tc":
            _check_meta_tc(meta, M, K)
            L.check(L.lib().s24_spmm(_p(v), _p(meta), _p(b), _p(c), M, N, K, b.stride(0), c.stride(0),
                                     _DT[vals.dtype], cfg, _stream(vals)))
        elif meta_layout == "ref":
            if meta.numel() != M * K // 16:
                raise RuntimeError(f"E has {meta.numel()} elements, expected {M * K // 16} for ({M}, {K})")
            if workspace is None:
                workspace = _new_meta_tc(M, K, vals.device)
            L.check(L.lib().s24_spmm_ref_meta(_p(v), _p(meta.contiguous()), _p(b), _p(c), M, N, K, b.stride(0),
                                              c.stride(0), _DT[vals.dtype], cfg, _p(workspace),
                                              workspace.numel() * 4, _stream(vals)))
        else:
            raise ValueError(f"unknown metadata layout {meta_layout!r}")
        _after_gemm(vals)
    return c


def spmm_prune_out(vals: torch.Tensor, meta: torch.Tensor, B: torch.Tensor, meta_layout: str = "tc",
                   want_ref: bool = True, want_tc: bool = False, manual_config: Optional[dict] = None):
    """Sparse GEMM whose epilogue 2:4-prunes and compresses the accumulator along N
    (compression/kernels/10.1_prune_acc.py:88-154,624-678): bit for bit prune + compress (signed keys,
    lower index on ties) of the C that `spmm` returns for the same operands and tile.

    Returns (C_vals (M, N/2), C_meta (M/16, N) int16 or None, C_meta_tc or None).
    """
    _require_cuda(vals, meta, B)
    M, N, K = _check_gemm(vals, B)
    if N % 128 != 0:
        raise RuntimeError(f"fused output prune needs N % 128 == 0 (got {N})")
    if meta_layout == "ref":
        meta_tc = meta_convert(meta, "ref", "tc", M, K)
    elif meta_layout == "tc":
        meta_tc = meta
        _check_meta_tc(meta_tc, M, K)
    else:
        raise ValueError(f"unknown metadata layout {meta_layout!r}")
    v = vals.contiguous()
    b = _row_major(B)
    cv = torch.empty((M, N // 2), dtype=vals.dtype, device=vals.device)
    ce = torch.empty((M // 16, N), dtype=torch.int16, device=vals.device) if want_ref else None
    ct = _new_meta_tc(M, N, vals.device) if want_tc else None
    with _on_device(vals):
        L.check(L.lib().s24_spmm_prune_out(_p(v), _p(meta_tc), _p(b), _p(cv), _p(ce), _p(ct), M, N, K,
                                           b.stride(0), _DT[vals.dtype], _tile_cfg(manual_config), _stream(vals)))
        _after_gemm(vals)
    return cv, ce, ct


def spmm_prune_in(A: torch.Tensor, B: torch.Tensor, mode: str = "signed", tie: str = "higher",
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = prune_2_4(A) @ B with the prune + compress of the dense A done inside the GEMM kernel
    (compression/kernels/7.8.1_prune_ws.py:112-192,609-650).  No compressed operand is materialised.

    The default tie rule is the reference kernel's (strict compare: the higher index survives equal
    keys); tie="reference" keeps the survivors of the torch function `prune_2_4` instead.
    """
    _require_cuda(A, B)
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[0]:
        raise RuntimeError(f"shapes do not chain: A {tuple(A.shape)}, B {tuple(B.shape)}")
    if A.dtype not in _DT or B.dtype != A.dtype:
        raise RuntimeError(f"A and B must both be float16 or bfloat16 (got {A.dtype}, {B.dtype})")
    M, K = A.shape
    N = B.shape[1]
    if M <= 0 or M % 32 != 0 or K <= 0 or K % 64 != 0 or N <= 0 or N % 8 != 0:
        raise RuntimeError(f"needs M % 32 == 0, K % 64 == 0, N % 8 == 0 (got M={M}, N={N}, K={K})")
    a = _row_major(A)
    b = _row_major(B)
    c = out if out is not None else torch.empty((M, N), dtype=A.dtype, device=A.device)
    if (tuple(c.shape) != (M, N) or c.dtype != A.dtype or c.device != A.device or c.stride(1) != 1
            or c.stride(0) % 8 != 0 or c.data_ptr() % 16 != 0):
        raise RuntimeError(f"`out` must be a ({M}, {N}) {A.dtype} tensor on {A.device} with unit column stride, "
                           "a row stride that is a multiple of 8 and 16-byte alignment")
    with _on_device(A):
        L.check(L.lib().s24_spmm_prune_in(_p(a), a.stride(0), _p(b), _p(c), M, N, K, b.stride(0), c.stride(0),
                                          _DT[A.dtype], _MODE[mode], _TIE[tie], _stream(A)))
        _after_gemm(A)
    return c


def spmm_scatter(vals: torch.Tensor, meta_tc: torch.Tensor, B: torch.Tensor, dst_ptrs, ldc: int) -> None:
    """C = A24 @ B stored to every address in `dst_ptrs` (1..8 device addresses of element (0, 0) of
    this product inside a destination with row stride `ldc`; this GPU's memory or peers' buffers
    opened with `peer_open`).  See s24_spmm_scatter; the caller orders the ranks afterwards."""
    _require_cuda(vals, meta_tc, B)
    M, N, K = _check_gemm(vals, B)
    dst_ptrs = [int(x) for x in dst_ptrs]
    if not 1 <= len(dst_ptrs) <= 8:
        raise RuntimeError(f"1 to 8 destinations (got {len(dst_ptrs)})")
    v = vals.contiguous()
    b = _row_major(B)
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    with _on_device(vals):
        _check_meta_tc(meta_tc, M, K)
        L.check(L.lib().s24_spmm_scatter(_p(v), _p(meta_tc), _p(b), arr, len(dst_ptrs), M, N, K, b.stride(0), int(ldc),
                                         _DT[vals.dtype], _stream(vals)))


def peer_alloc(nbytes: int, device: torch.device) -> int:
    """exportable device memory on `device` (cudaMalloc; set-up code only)"""
    out = ctypes.c_void_p()
    with torch.cuda.device(device):
        L.check(L.lib().s24_peer_alloc(int(nbytes), ctypes.byref(out)))
    return int(out.value)


def peer_free(ptr: int) -> None:
    L.check(L.lib().s24_peer_free(ctypes.c_void_p(ptr)))


def peer_export(ptr: int) -> bytes:
    buf = ctypes.create_string_buffer(L.PEER_HANDLE_BYTES)
    L.check(L.lib().s24_peer_export(ctypes.c_void_p(ptr), buf))
    return buf.raw


def peer_open(handle: bytes, device: torch.device) -> int:
    """map another process's exported buffer; `device` is the GPU whose kernels will store to it"""
    if len(handle) != L.PEER_HANDLE_BYTES:
        raise RuntimeError(f"a peer handle has {L.PEER_HANDLE_BYTES} bytes (got {len(handle)})")
    out = ctypes.c_void_p()
    with torch.cuda.device(device):
        L.check(L.lib().s24_peer_open(ctypes.create_string_buffer(handle, L.PEER_HANDLE_BYTES), ctypes.byref(out)))
    return int(out.value)


def peer_close(ptr: int) -> None:
    L.check(L.lib().s24_peer_close(ctypes.c_void_p(ptr)))


def peer_copy_2d(dst_ptr: int, dst_pitch: int, src_ptr: int, src_pitch: int, width_bytes: int, rows: int,
                 stream: torch.cuda.Stream) -> None:
    """enqueue a pitched block copy (copy engines) on `stream`; dst may be a peer mapping"""
    L.check(L.lib().s24_peer_copy_2d(ctypes.c_void_p(dst_ptr), int(dst_pitch), ctypes.c_void_p(src_ptr), int(src_pitch),
                                     int(width_bytes), int(rows), ctypes.c_void_p(stream.cuda_stream)))


def relayout_shards(stage: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """stage (G, rows, nl) shard-major -> out (rows, G * nl) row-major (see s24_relayout_shards)."""
    _require_cuda(stage, out)
    G, rows, nl = stage.shape
    if not stage.is_contiguous() or stage.element_size() != 2 or out.element_size() != 2:
        raise RuntimeError("relayout_shards needs a contiguous 16-bit (G, rows, nl) stage")
    if tuple(out.shape) != (rows, G * nl) or out.stride(1) != 1:
        raise RuntimeError(f"`out` must be ({rows}, {G * nl}) with unit column stride")
    with _on_device(stage):
        L.check(L.lib().s24_relayout_shards(_p(stage), _p(out), rows, G, nl, out.stride(0), _stream(stage)))
    return out
