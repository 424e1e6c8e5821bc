"""CPU oracle of the TN GEMM path.  TEST INFRASTRUCTURE ONLY - never on the product path.

Two independent restatements of the reference's ground truth:

* ``reference_matmul_fp32`` - the reference's own check expression,
  ``torch.matmul(A.float(), B.float().T)`` (kernels/tests/gemm_test.py:36), on CPU.
* ``c_gemm_tn_f32`` / ``c_gemm_tn`` - the plain-C restatement in gemm_oracle.c (fp32 products
  and sums, then round-to-nearest-even to the 16-bit type, the conversion the reference fuses
  into its epilogue, kernels/gemm_kernels/sm90a/gemm.cuh:368-377).

plus the two acceptance metrics: the reference's ``allclose(atol=1e-2, rtol=1e-2)``
(``measure_error_stats``, kernels/tests/gemm_test.py:4-11) and the normalised maximum error
``max|C - C_ref| / max|C_ref|`` (<= 2e-2 for bf16 output, <= 5e-3 for fp16 output).

Parity status: the reference ships no golden vectors for this path.  Both restatements are
pinned against tests/golden/gemm_tn_golden.npz, which tests/golden/make_golden.py generated in
the build container by evaluating the reference's check expression (and its
``measure_error_stats``, imported from the reference tree) on seeded inputs.  Bitwise parity
with the reference's Hopper kernel is not obtainable (its summation order is the wgmma
hardware's and it cannot run on sm_100); parity is at the stated tolerances.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import time
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libgemm_oracle.so"

TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1}


# ------------------------------------------------------------------ inputs ---
def make_inputs(M: int, N: int, K: int, seed: int, dtype=torch.bfloat16, a_std: float | None = None,
                b_std: float | None = None):
    """Seeded operands on the CPU: fp32 normal draws (A first, then B, one generator), scaled,
    then cast to `dtype`.  `a_std` / `b_std` default to 1/sqrt(K) (the square-GEMM configs);
    the MLP and small-M configs use a_std=1, b_std=0.02.  The reference draws unseeded N(0,1)
    (kernels/tests/gemm_test.py:23-24)."""
    g = torch.Generator().manual_seed(seed)
    sa = (1.0 / K ** 0.5) if a_std is None else a_std
    sb = (1.0 / K ** 0.5) if b_std is None else b_std
    A = (torch.randn(M, K, generator=g, dtype=torch.float32) * sa).to(dtype)
    B = (torch.randn(N, K, generator=g, dtype=torch.float32) * sb).to(dtype)
    return A, B


def make_ternary_inputs(M: int, N: int, K: int, seed: int, dtype=torch.bfloat16):
    """A, B with entries in {-1, 0, 1}: for K <= 256 every partial sum is a small integer,
    exact in fp32 and in the 16-bit output, so any correct kernel must match BITWISE."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-1, 2, (M, K), generator=g).to(dtype)
    B = torch.randint(-1, 2, (N, K), generator=g).to(dtype)
    return A, B


# ------------------------------------------------- the reference's check ---
def reference_matmul_fp32(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """Ground truth exactly as the reference computes it (kernels/tests/gemm_test.py:36)."""
    return torch.matmul(A.float(), B.float().T)


def measure_error_stats(pred: torch.Tensor, label: torch.Tensor):
    """Restates kernels/tests/gemm_test.py:4-11 without the prints: (max, mean) absolute error
    and whether allclose(atol=1e-2, rtol=1e-2) holds."""
    abs_diff = torch.abs(pred - label)
    ok = torch.allclose(pred, label, atol=1e-2, rtol=1e-2)
    return abs_diff.max().item(), abs_diff.mean().item(), ok


def normalized_max_error(C: torch.Tensor, C_ref: torch.Tensor) -> float:
    """max|C - C_ref| / max|C_ref| in fp32 (the acceptance metric of this build)."""
    C = C.detach().float().cpu()
    C_ref = C_ref.detach().float().cpu()
    denom = C_ref.abs().max().item()
    if denom == 0.0:
        return float((C - C_ref).abs().max().item())
    return float((C - C_ref).abs().max().item() / denom)


def tolerance(dtype) -> float:
    return TOL[dtype]


# ----------------------------------------------------- the C restatement ---
def build(force: bool = False) -> Path:
    src = HERE / "gemm_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B" if force else "-s"], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def _load():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        lib = ctypes.CDLL(str(LIB_PATH))
        L, P, I = ctypes.c_long, ctypes.c_void_p, ctypes.c_int
        lib.oracle_gemm_tn_f32.argtypes = [P, P, P, L, L, L, L, L, L, I]
        lib.oracle_gemm_tn_f32.restype = I
        lib.oracle_gemm_tn.argtypes = [P, P, P, L, L, L, L, L, L, I]
        lib.oracle_gemm_tn.restype = I
        lib.oracle_round_to_16.argtypes = [P, P, L, I]
        lib.oracle_round_to_16.restype = I
        lib.oracle_widen_16.argtypes = [P, P, L, I]
        lib.oracle_widen_16.restype = I
        _lib = lib
    return _lib


def _bits(t: torch.Tensor) -> torch.Tensor:
    assert t.dtype in DTYPE_CODE and t.device.type == "cpu"
    return t.contiguous().view(torch.int16)


def c_gemm_tn_f32(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """fp32 A @ B.T by the C restatement (CPU tensors of bf16 / fp16)."""
    lib = _load()
    M, K = A.shape
    N = B.shape[0]
    a, b = _bits(A), _bits(B)
    C = torch.empty((M, N), dtype=torch.float32)
    rc = lib.oracle_gemm_tn_f32(a.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, K, K, N, DTYPE_CODE[A.dtype])
    if rc != 0:
        raise RuntimeError("oracle_gemm_tn_f32 failed")
    return C


def c_gemm_tn(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """RN-rounded 16-bit A @ B.T by the C restatement."""
    lib = _load()
    M, K = A.shape
    N = B.shape[0]
    a, b = _bits(A), _bits(B)
    C = torch.empty((M, N), dtype=torch.int16)
    rc = lib.oracle_gemm_tn(a.data_ptr(), b.data_ptr(), C.data_ptr(), M, N, K, K, K, N, DTYPE_CODE[A.dtype])
    if rc != 0:
        raise RuntimeError("oracle_gemm_tn failed")
    return C.view(A.dtype)


def c_round_to_16(x: torch.Tensor, dtype) -> torch.Tensor:
    lib = _load()
    x = x.contiguous().float()
    out = torch.empty(x.shape, dtype=torch.int16)
    if lib.oracle_round_to_16(x.data_ptr(), out.data_ptr(), x.numel(), DTYPE_CODE[dtype]) != 0:
        raise RuntimeError("oracle_round_to_16 failed")
    return out.view(dtype)


def c_widen_16(x: torch.Tensor) -> torch.Tensor:
    lib = _load()
    bits = _bits(x)
    out = torch.empty(x.shape, dtype=torch.float32)
    if lib.oracle_widen_16(bits.data_ptr(), out.data_ptr(), x.numel(), DTYPE_CODE[x.dtype]) != 0:
        raise RuntimeError("oracle_widen_16 failed")
    return out


# ------------------------------------------------------------ CPU timing ---
def time_cpu_matmul(A: torch.Tensor, B: torch.Tensor, min_seconds: float = 0.0, max_runs: int = 3):
    """Times the reference check expression on the host cores.  Returns (seconds per call,
    threads used, result of the last call)."""
    out = reference_matmul_fp32(A, B)  # warm-up (thread pool, page faults)
    runs, total = 0, 0.0
    while runs < max_runs and (runs == 0 or total < min_seconds):
        t0 = time.perf_counter()
        out = reference_matmul_fp32(A, B)
        total += time.perf_counter() - t0
        runs += 1
    return total / runs, torch.get_num_threads(), out
