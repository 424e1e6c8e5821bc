"""gemm_kernels: B200 (sm_100a) TN GEMM behind the reference's Python entry point.

``gemm_tn_test(A, B, C)`` computes ``C[M,N] = A[M,K] @ B[N,K].T`` (bf16 or fp16 inputs,
fp32 accumulation, same-dtype output), writes it into the caller's ``C`` and returns ``C``:
the contract of the reference's ``gemm_kernels._C.gemm_tn_test``
(kernels/gemm_kernels/__init__.cpp:6-9, kernels/gemm_kernels/sm90a/gemm_test.cu:12-92).

The reference's package ``__init__.py`` is empty, so its own scripts'
``from gemm_kernels import gemm_tn_test`` (kernels/tests/gemm_test.py:2) cannot resolve;
this module re-exports the symbol so that import works, and keeps ``gemm_kernels._C``.

There is no CPU or eager fallback: importing this package without the compiled extension
raises ImportError with the build command.
"""
from __future__ import annotations

import os as _os

try:
    from . import _C  # noqa: F401
except ImportError as exc:  # pragma: no cover - exercised only on an unbuilt tree
    _here = _os.path.dirname(_os.path.abspath(__file__))
    raise ImportError(
        "gemm_kernels._C is not built (sm_100a only, no fallback path). Build it in-tree with "
        f"`python {_os.path.join(_os.path.dirname(_here), 'build_native.py')}`"
    ) from exc

import torch as _torch

gemm_tn_test = _C.gemm_tn_test
gemm_tn_fanout = _C.gemm_tn_fanout
device_status = _C.device_status
init = _C.init
set_option = _C.set_option
set_trace_buffer = _C.set_trace_buffer
describe_config = _C.describe_config
describe_plan = _C.describe_plan
select_config = _C.select_config
workspace_bytes = _C.workspace_bytes
num_sms = _C.num_sms

LIBRARY_PATH = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "libgemm_sm100.so")

DTYPE_CODES = {_torch.bfloat16: 0, _torch.float16: 1}


def trace_launch(A: "_torch.Tensor", B: "_torch.Tensor", C: "_torch.Tensor") -> dict:
    """Runs ``gemm_tn_test(A, B, C)`` once with the per-CTA trace counters on and returns
    ``{"cycles": mean SM cycles from kernel entry to exit, "ns": mean wall time of a CTA,
    "sm_mhz": cycles / ns * 1000}``.  The cycle count does not depend on the clock, so
    ``cycles / (measured seconds per launch)`` gives the clock a timed run really had; the
    driver-reported clock does not follow the fast power-management steps of a power-capped GPU."""
    trace = _torch.zeros(num_sms() * 16, dtype=_torch.int64, device=A.device)
    set_trace_buffer(trace)
    try:
        gemm_tn_test(A, B, C)
        _torch.cuda.synchronize(A.device)
    finally:
        set_trace_buffer(None)
    t = trace.view(-1, 16).cpu()
    used = t[:, 13] > t[:, 12]
    if not bool(used.any()):
        return {"cycles": float("nan"), "ns": float("nan"), "sm_mhz": float("nan")}
    cycles = (t[used, 10] - t[used, 0]).double()
    ns = (t[used, 13] - t[used, 12]).double()
    return {"cycles": float(cycles.mean().item()), "ns": float(ns.mean().item()),
            "sm_mhz": float((cycles / ns).mean().item() * 1000.0)}


def gemm_tn(A: "_torch.Tensor", B: "_torch.Tensor", out: "_torch.Tensor | None" = None) -> "_torch.Tensor":
    """``A[M,K] @ B[N,K].T`` into ``out`` (allocated as ``[M,N]`` of A's dtype when None)."""
    if out is None:
        out = _torch.empty((A.shape[0], B.shape[0]), dtype=A.dtype, device=A.device)
    return gemm_tn_test(A, B, out)


def gemm_nn(A: "_torch.Tensor", B: "_torch.Tensor", out: "_torch.Tensor | None" = None) -> "_torch.Tensor":
    """``A[M,K] @ B[K,N]`` (B as ``torch.mm`` takes it) into ``out``; no transposed copy of B."""
    if out is None:
        out = _torch.empty((A.shape[0], B.shape[1]), dtype=A.dtype, device=A.device)
    return _C.gemm_nn(A, B, out)


def gemm(A: "_torch.Tensor", B: "_torch.Tensor", out: "_torch.Tensor | None" = None, a_is_km: bool = False,
         b_is_kn: bool = True, alpha: float = 1.0, beta: float = 0.0) -> "_torch.Tensor":
    """``alpha * op(A) @ op(B) + beta * out`` for all four operand layouts without transposed copies:
    A is ``[M,K]`` or, with ``a_is_km``, ``[K,M]``; B is ``[K,N]`` (the default, as ``torch.mm`` takes
    it) or, with ``b_is_kn=False``, ``[N,K]`` (the layout of ``gemm_tn_test``).  ``alpha`` and ``beta``
    are applied to the fp32 accumulator before the one rounding to the output type (``torch.addmm``
    semantics); ``beta != 0`` needs ``out``."""
    M = A.shape[1] if a_is_km else A.shape[0]
    N = B.shape[1] if b_is_kn else B.shape[0]
    if out is None:
        if beta != 0.0:
            raise ValueError("beta != 0 reads `out`: pass it")
        out = _torch.empty((M, N), dtype=A.dtype, device=A.device)
    return _C.gemm_layouts(A, B, out, a_is_km, b_is_kn, alpha, beta)


class HostGemm:
    """``C_host = A_host @ B_host.T`` for operands and result in (pinned) HOST memory.

    The whole of B is uploaded first; A is uploaded in row panels, each panel's GEMM starts as
    soon as its rows have arrived, and each finished panel of C goes back to the host while the
    next panel of A is still coming in (PCIe carries both directions at once).  The upload link
    is busy from the first byte to the last, so the step takes the upload time plus what follows
    the last byte of A: the last panel's GEMM and download.  The last of the `panels` panels is
    therefore cut once more into quarters.  Device buffers and streams are created once and
    reused; `__call__` returns after the last byte of C has reached the host.  The reference has
    no host-memory path: its callers create operands on the device (kernels/tests/gemm_test.py:23-28).
    """

    def __init__(self, M: int, N: int, K: int, dtype=_torch.bfloat16, device="cuda", panels: int = 8):
        self.M, self.N, self.K = M, N, K
        self.device = _torch.device(device)
        rows = -(-M // max(1, panels))
        self.panel_rows = max(256, -(-rows // 256) * 256) if M >= 256 else M
        # row ranges: equal panels, the last one in quarters (multiples of 256 rows where possible)
        self.ranges = []
        for r0 in range(0, M, self.panel_rows):
            r1 = min(M, r0 + self.panel_rows)
            if r1 == M and r1 - r0 >= 1024:
                q = -(-(r1 - r0) // 4 // 256) * 256
                self.ranges += [(a, min(M, a + q)) for a in range(r0, r1, q)]
            else:
                self.ranges.append((r0, r1))
        self.A = _torch.empty((M, K), dtype=dtype, device=self.device)
        self.B = _torch.empty((N, K), dtype=dtype, device=self.device)
        self.C = _torch.empty((M, N), dtype=dtype, device=self.device)
        self.h2d = _torch.cuda.Stream(device=self.device)
        self.d2h = _torch.cuda.Stream(device=self.device)

    def __call__(self, A_host: "_torch.Tensor", B_host: "_torch.Tensor", C_host: "_torch.Tensor") -> "_torch.Tensor":
        if tuple(A_host.shape) != (self.M, self.K) or tuple(B_host.shape) != (self.N, self.K) or \
                tuple(C_host.shape) != (self.M, self.N):
            raise ValueError("operand shapes do not match the plan")
        compute = _torch.cuda.current_stream(self.device)
        self.h2d.wait_stream(compute)          # the previous call's kernels are done with A and B
        self.d2h.wait_stream(compute)
        with _torch.cuda.stream(self.h2d):
            self.B.copy_(B_host, non_blocking=True)
        for r0, r1 in self.ranges:
            with _torch.cuda.stream(self.h2d):
                self.A[r0:r1].copy_(A_host[r0:r1], non_blocking=True)
                arrived = _torch.cuda.Event()
                arrived.record(self.h2d)
            compute.wait_event(arrived)
            gemm_tn_test(self.A[r0:r1], self.B, self.C[r0:r1])
            done = _torch.cuda.Event()
            done.record(compute)
            self.d2h.wait_event(done)
            with _torch.cuda.stream(self.d2h):
                C_host[r0:r1].copy_(self.C[r0:r1], non_blocking=True)
        compute.wait_stream(self.d2h)
        compute.synchronize()
        return C_host


from .nsplit import FusedNSplit, NSplitPlan, fanout_pointers, gemm_tn_nsplit, shard_rows  # noqa: E402

__all__ = [
    "gemm_tn_test", "gemm_tn", "gemm_nn", "gemm", "HostGemm", "gemm_tn_fanout", "gemm_tn_nsplit", "FusedNSplit", "NSplitPlan", "shard_rows", "device_status",
    "init", "set_option", "set_trace_buffer", "trace_launch", "describe_config", "describe_plan", "select_config", "workspace_bytes", "num_sms", "LIBRARY_PATH",
]
