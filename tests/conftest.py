"""Shared test plumbing: the `gpu` marker, import paths, the golden fixture and the C ABI."""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parents[1]
PKG_ROOT = REPO / "cute-examples_b200"
for p in (str(REPO), str(PKG_ROOT)):
    if p not in sys.path:
        sys.path.insert(0, p)

LIB_PATH = PKG_ROOT / "gemm_kernels" / "libgemm_sm100.so"
HEADER = REPO / "include" / "gemm_sm100.h"
GOLDEN = REPO / "tests" / "golden" / "gemm_tn_golden.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU; run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


def load_capi() -> ctypes.CDLL:
    """The C ABI of include/gemm_sm100.h through ctypes, with prototypes set."""
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is not built; run python cute-examples_b200/build_native.py")
    lib = ctypes.CDLL(str(LIB_PATH))
    I, L, P, Z = ctypes.c_int, ctypes.c_long, ctypes.c_void_p, ctypes.c_size_t
    lib.gemm_sm100_tn.argtypes = [P, P, P, I, I, I, L, L, L, I, P, Z, P, ctypes.POINTER(I)]
    lib.gemm_sm100_tn.restype = I
    lib.gemm_sm100_nn.argtypes = [P, P, P, I, I, I, L, L, L, I, P, ctypes.POINTER(I)]
    lib.gemm_sm100_nn.restype = I
    lib.gemm_sm100_gemm.argtypes = [P, P, P, I, I, I, L, L, L, I, I, I, P, ctypes.POINTER(I)]
    lib.gemm_sm100_gemm.restype = I
    lib.gemm_sm100_gemm_scaled.argtypes = [P, P, P, I, I, I, L, L, L, I, I, I, ctypes.c_float, ctypes.c_float, P,
                                           ctypes.POINTER(I)]
    lib.gemm_sm100_gemm_scaled.restype = I
    lib.gemm_sm100_tn_fanout.argtypes = [P, P, ctypes.POINTER(P), I, I, I, I, L, L, L, I, P, ctypes.POINTER(I)]
    lib.gemm_sm100_tn_fanout.restype = I
    lib.gemm_sm100_tn_static_scratch.argtypes = [P, P, P, I, I, I, L, L, L, I, P, ctypes.POINTER(I)]
    lib.gemm_sm100_tn_static_scratch.restype = I
    lib.gemm_sm100_static_scratch_capacity.argtypes = []
    lib.gemm_sm100_static_scratch_capacity.restype = Z
    lib.gemm_sm100_workspace_bytes.argtypes = [I, I, I, I]
    lib.gemm_sm100_workspace_bytes.restype = Z
    lib.gemm_sm100_workspace_register.argtypes = [P, Z, P, ctypes.POINTER(I)]
    lib.gemm_sm100_workspace_register.restype = I
    lib.gemm_sm100_workspace_unregister.argtypes = [P]
    lib.gemm_sm100_workspace_unregister.restype = I
    lib.gemm_sm100_resident_clusters.argtypes = [I]
    lib.gemm_sm100_resident_clusters.restype = I
    lib.gemm_sm100_num_sms.argtypes = []
    lib.gemm_sm100_num_sms.restype = I
    lib.gemm_sm100_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(I)]
    lib.gemm_sm100_device_status.restype = I
    lib.gemm_sm100_set_option.argtypes = [ctypes.c_char_p, L]
    lib.gemm_sm100_set_option.restype = I
    lib.gemm_sm100_describe_config.argtypes = [I, ctypes.c_char_p, Z]
    lib.gemm_sm100_describe_config.restype = I
    lib.gemm_sm100_describe_plan.argtypes = [I, I, I, I, ctypes.c_char_p, Z]
    lib.gemm_sm100_describe_plan.restype = I
    lib.gemm_sm100_select_config.argtypes = [I, I, I, I]
    lib.gemm_sm100_select_config.restype = I
    lib.gemm_sm100_selftest_wait_timeout.argtypes = [P, ctypes.POINTER(I)]
    lib.gemm_sm100_selftest_wait_timeout.restype = I
    lib.gemm_sm100_set_trace_buffer.argtypes = [P, Z]
    lib.gemm_sm100_set_trace_buffer.restype = I
    lib.gemm_sm100_init.argtypes = [ctypes.POINTER(I)]
    lib.gemm_sm100_init.restype = I
    lib.gemm_sm100_error_string.argtypes = [I]
    lib.gemm_sm100_error_string.restype = ctypes.c_char_p
    return lib


@pytest.fixture(scope="session")
def capi():
    return load_capi()


def capi_gemm(lib, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, ldc: int | None = None) -> int:
    """Calls gemm_sm100_tn on CUDA tensors with raw pointers; returns the status code."""
    M, K = A.shape
    N = B.shape[0]
    dtype = {torch.bfloat16: 0, torch.float16: 1}[A.dtype]
    ws_bytes = lib.gemm_sm100_workspace_bytes(M, N, K, dtype)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=A.device) if ws_bytes else None
    err = ctypes.c_int(0)
    stream = torch.cuda.current_stream(A.device).cuda_stream
    rc = lib.gemm_sm100_tn(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, A.stride(0) if M > 1 else K,
                           B.stride(0) if N > 1 else K, ldc if ldc is not None else (C.stride(0) if M > 1 else N),
                           dtype, ws.data_ptr() if ws is not None else None, ws_bytes, stream, ctypes.byref(err))
    return rc


def capi_status(lib) -> tuple[int, int]:
    word = ctypes.c_uint(0)
    err = ctypes.c_int(0)
    rc = lib.gemm_sm100_device_status(ctypes.byref(word), ctypes.byref(err))
    return rc, word.value
