"""The C-ABI library loads without a GPU and exports every symbol include/s24.h declares."""
import ctypes
import re
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "gpu-compression-kernel_b200"
sys.path.insert(0, str(PKG))


@pytest.fixture(scope="module")
def built():
    sys.path.insert(0, str(PKG))
    import build as s24_build
    return s24_build.build()


def declared_symbols():
    text = (ROOT / "include" / "s24.h").read_text()
    return sorted(set(re.findall(r"S24_API[^;(]*?\b(s24_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for want in ("s24_version", "s24_last_error", "s24_prune", "s24_compress", "s24_prune_compress",
                 "s24_meta_tc_bytes", "s24_meta_convert", "s24_spmm", "s24_spmm_ref_meta", "s24_spmm_ref_meta_noalloc", "s24_spmm_prune_out",
                 "s24_device_status", "s24_relayout_shards", "s24_spmm_bt", "s24_spmm_prune_in", "s24_spmm_scatter",
                 "s24_peer_alloc", "s24_peer_free", "s24_peer_export", "s24_peer_open", "s24_peer_close"):
        assert want in names


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(str(built))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in include/s24.h but not exported"


def test_ctypes_signatures_cover_the_header(built):
    from s24 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    L = _lib.lib()
    assert L.s24_version() == 1
    assert L.s24_meta_tc_bytes(256, 512) == 256 * 512 // 8
    assert L.s24_meta_tc_bytes(160, 192) == 2 * 2 * 2048       # whole (128-row, 128-column) records


def test_argument_errors_need_no_gpu(built):
    # validation happens before any CUDA call, so it can be exercised on a CPU-only box
    from s24 import _lib
    L = _lib.lib()
    assert L.s24_prune(None, None, 8, 0, 0, 0, None) == _lib.ERR_INVALID_ARG
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert L.s24_prune(p, p, 6, 0, 0, 0, None) == _lib.ERR_SHAPE
    assert "divisible by 4" in _lib.last_error()
    assert L.s24_prune_compress(p, 48, 64, 64, 0, 0, 0, p, p, None, None) == _lib.ERR_SHAPE
    assert "divisible by 32" in _lib.last_error()
    assert L.s24_prune_compress(p, 32, 80, 80, 0, 0, 0, p, p, None, None) == _lib.ERR_SHAPE
    assert L.s24_prune_compress(p, 32, 64, 64, 7, 0, 0, p, p, None, None) == _lib.ERR_INVALID_ARG
    assert L.s24_spmm(p, p, p, p, 100, 128, 128, 128, 128, 0, None, None) == _lib.ERR_SHAPE
    assert L.s24_meta_convert(p, 1, p, 2, 48, 128, None) == _lib.ERR_SHAPE          # M % 32
    assert L.s24_spmm(p, p, p, p, 128, 128, 96, 128, 128, 0, None, None) == _lib.ERR_SHAPE   # K % 64


def test_cpu_tensors_are_rejected_loudly(built):
    import torch
    import s24
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        s24.prune(torch.zeros(4, 8, dtype=torch.float16))
    with pytest.raises(ValueError):
        s24.prune(torch.zeros(4, 6, dtype=torch.float16))


def test_more_argument_errors_need_no_gpu(built):
    """entry points added for the multi-GPU and self-test paths validate before touching CUDA too"""
    from s24 import _lib
    L = _lib.lib()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert L.s24_peer_copy_2d(None, 64, p, 64, 32, 4, None) == _lib.ERR_INVALID_ARG
    assert L.s24_peer_copy_2d(p, 16, p, 64, 32, 4, None) == _lib.ERR_SHAPE           # pitch smaller than the width
    assert L.s24_peer_copy_2d(p, 64, p, 64, 0, 4, None) == _lib.OK                   # nothing to copy
    assert L.s24_selftest_timeout(5, None, None, None, None, 0, 0, 0, 0, None, None) == _lib.ERR_INVALID_ARG
    assert L.s24_selftest_timeout(1, p, p, p, p, 128, 128, 128, 0, None, None) == _lib.ERR_SHAPE   # needs two k-blocks
    # shapes of the reference-layout entry points are checked before their scratch is sized
    assert L.s24_spmm_ref_meta_noalloc(p, p, p, p, 1 << 40, 128, 1 << 40, 128, 128, 0, None, None) == _lib.ERR_SHAPE
    assert L.s24_spmm_ref_meta_noalloc(p, p, p, p, 16384, 128, 16384, 128, 128, 0, None, None) == _lib.ERR_SHAPE
    assert "built-in buffer" in _lib.last_error()


def test_library_path_can_be_overridden(built, tmp_path):
    """S24_LIBRARY=<path> loads another build of the library (variant builds of build.py --define ... --out ...)"""
    import shutil
    import subprocess
    other = tmp_path / "libs24_copy.so"
    shutil.copy(built, other)
    code = ("import sys; sys.path.insert(0, %r); from s24 import _lib; "
            "assert str(_lib.LIB_PATH) == %r, _lib.LIB_PATH; assert _lib.lib().s24_version() == 1; print('ok')" % (str(PKG), str(other)))
    import os
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, S24_LIBRARY=str(other)), capture_output=True, text=True)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


def test_a_c_program_binds_the_library(built, tmp_path):
    """gcc compiles tests/host/abi_smoke.c against include/s24.h, links libs24.so and runs it: the
    boundary is plain C (no C++ types, no torch), and its argument validation needs no GPU"""
    import subprocess
    exe = tmp_path / "abi_smoke"
    libdir = built.parent
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", f"-I{ROOT / 'include'}", str(ROOT / "tests/host/abi_smoke.c"),
                    "-o", str(exe), f"-L{libdir}", "-ls24", f"-Wl,-rpath,{libdir}"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "abi smoke ok" in r.stdout, r.stdout + r.stderr
