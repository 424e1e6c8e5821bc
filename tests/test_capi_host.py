"""The C-ABI library without a GPU: it loads, exports every symbol the header declares, and
rejects bad arguments before touching CUDA."""
import ctypes
import re

import pytest
import torch

from conftest import HEADER, LIB_PATH, load_capi


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(gemm_sm100_\w+)\s*\(", text)))


def test_library_is_built():
    assert LIB_PATH.exists(), "build with: python cute-examples_b200/build_native.py"


def test_every_declared_symbol_is_exported(capi):
    names = declared_symbols()
    assert "gemm_sm100_tn" in names and len(names) >= 8
    for n in names:
        assert hasattr(capi, n), f"{n} declared in include/gemm_sm100.h but not exported"


def test_error_strings(capi):
    for code in range(0, 10):
        s = capi.gemm_sm100_error_string(code)
        assert s and s != b"unknown error code"
    assert capi.gemm_sm100_error_string(12345) == b"unknown error code"


def test_describe_and_options(capi):
    buf = ctypes.create_string_buffer(256)
    n = 0
    while capi.gemm_sm100_describe_config(n, buf, 256) == 0:
        assert b"tile=" in buf.value and b"stages=" in buf.value
        n += 1
    assert n >= 4
    assert b"epilogue_warps=" in buf.value
    assert capi.gemm_sm100_set_option(b"tile_config", n) == 9
    assert capi.gemm_sm100_set_option(b"tile_config", -1) == 0
    assert capi.gemm_sm100_set_option(b"timeout_ms", 0) == 9
    assert capi.gemm_sm100_set_option(b"timeout_ms", 2000) == 0
    assert capi.gemm_sm100_set_option(b"no_such_option", 1) == 9
    assert capi.gemm_sm100_set_option(None, 1) == 1


BAD = [
    # M, N, K, lda, ldb, ldc, dtype, a, b, c, expected
    (-1, 8, 8, 8, 8, 8, 0, 256, 512, 1024, 2),       # negative extent
    (8, 8, 8, 8, 8, 8, 7, 256, 512, 1024, 4),        # dtype
    (8, 8, 12, 16, 16, 8, 0, 256, 512, 1024, 2),     # K % 8
    (8, 8, 16, 8, 16, 8, 0, 256, 512, 1024, 2),      # lda < K
    (8, 16, 16, 16, 16, 8, 0, 256, 512, 1024, 2),    # ldc < N
    (8, 8, 16, 20, 16, 8, 0, 256, 512, 1024, 3),     # lda % 8
    (8, 8, 16, 16, 16, 8, 0, 260, 512, 1024, 3),     # A misaligned
    (8, 8, 16, 16, 16, 8, 0, 256, 512, 1028, 3),     # C misaligned
    (8, 8, 16, 16, 16, 8, 0, 0, 512, 1024, 1),       # null A
    (8, 8, 16, 16, 16, 8, 0, 256, 512, 0, 1),        # null C
]


@pytest.mark.parametrize("case", BAD)
def test_bad_arguments_are_rejected_on_the_host(capi, case):
    M, N, K, lda, ldb, ldc, dtype, a, b, c, want = case
    err = ctypes.c_int(-7)
    rc = capi.gemm_sm100_tn(a or None, b or None, c or None, M, N, K, lda, ldb, ldc, dtype, None, 0, None,
                            ctypes.byref(err))
    assert rc == want
    assert err.value == 0


def test_empty_problem_is_a_noop(capi):
    err = ctypes.c_int(0)
    assert capi.gemm_sm100_tn(None, None, None, 0, 8, 8, 8, 8, 8, 0, None, 0, None, ctypes.byref(err)) == 0
    assert capi.gemm_sm100_tn(None, None, None, 8, 0, 8, 8, 8, 8, 0, None, 0, None, ctypes.byref(err)) == 0


def test_scaled_entry_validates_on_the_host(capi):
    err = ctypes.c_int(0)
    # K == 0 with beta != 0 would be "C *= beta", which is not this library's job.
    assert capi.gemm_sm100_gemm_scaled(256, 512, 1024, 8, 8, 0, 8, 8, 8, 0, 0, 0, 1.0, 0.5, None,
                                       ctypes.byref(err)) == 2
    assert capi.gemm_sm100_gemm_scaled(256, 512, 1024, 8, 8, 12, 16, 16, 8, 0, 0, 0, 2.0, 0.0, None,
                                       ctypes.byref(err)) == 2
    assert capi.gemm_sm100_gemm_scaled(None, None, None, 0, 8, 8, 8, 8, 8, 0, 0, 1, 2.0, 1.0, None,
                                       ctypes.byref(err)) == 0


def test_binding_rejects_bad_tensors_with_runtime_error():
    """Shape and dtype checks of the binding need no device: wrong dtype, K mismatch, wrong rank,
    wrong C shape, strided K all raise RuntimeError (the reference's TORCH_CHECKs,
    gemm_test.cu:15-41), and CPU tensors are refused last."""
    import gemm_kernels as gk

    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt)  # noqa: E731
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        gk.gemm_tn_test(z(8, 8), z(8, 8), z(8, 8))
    with pytest.raises(RuntimeError, match=r"Inner dimensions of A and B must match \(A: 64, B: 128\)"):
        gk.gemm_tn_test(z(64, 64), z(64, 128), z(64, 64))
    with pytest.raises(RuntimeError, match="same dtype"):
        gk.gemm_tn_test(z(64, 64), z(64, 64, dt=torch.float16), z(64, 64))
    with pytest.raises(RuntimeError, match="bfloat16 or float16"):
        gk.gemm_tn_test(*(z(64, 64, dt=torch.float32),) * 3)
    with pytest.raises(RuntimeError, match="2D"):
        gk.gemm_tn_test(z(64), z(64, 64), z(64, 64))
    with pytest.raises(RuntimeError, match="shape"):
        gk.gemm_tn_test(z(64, 64), z(32, 64), z(64, 64))
    with pytest.raises(RuntimeError, match="contiguous along K"):
        gk.gemm_tn_test(z(64, 128)[:, ::2], z(64, 64), z(64, 64))
    with pytest.raises(RuntimeError, match="unit stride"):
        gk.gemm_tn_test(z(64, 64), z(64, 64), z(64, 128)[:, ::2])
    assert gk.gemm_tn_test is gk._C.gemm_tn_test
    # keyword names of the reference binding
    with pytest.raises(RuntimeError):
        gk.gemm_tn_test(A=z(8, 8), B=z(8, 8), C=z(8, 8))


def test_environment_overrides_are_read_at_load():
    """A fresh process that sets GEMM_SM100_TILE_CONFIG sees it as the initial option value:
    select_config then returns that configuration whatever the shape."""
    import os
    import subprocess
    import sys

    code = ("import ctypes;"
            f"lib = ctypes.CDLL({str(LIB_PATH)!r});"
            "lib.gemm_sm100_select_config.argtypes = [ctypes.c_int] * 4;"
            "print(lib.gemm_sm100_select_config(8192, 8192, 8192, 0), lib.gemm_sm100_select_config(128, 256, 64, 0))")
    env = dict(os.environ, GEMM_SM100_TILE_CONFIG="2")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout.split()
    assert out == ["2", "2"]
    env = dict(os.environ, GEMM_SM100_TILE_CONFIG="99")           # out of range: ignored
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, check=True).stdout.split()
    assert out[0] in ("0", "1")           # the planner's own choice for a large square: a pair tile
