"""gemm_sm100_tn_static_scratch: the entry point for hosts that cannot give the library scratch
memory and must not see it allocate (it keeps its K-split counters and partial tiles in an
array built into the library).  Collected last on purpose: a run that stops at the first failure
has then already run everything else.

Checked through the C ABI, on two calls in a row that share the built-in array:
  * against gemm_sm100_tn forced onto the same kernel and schedule with a caller workspace
    (same arithmetic in the same order: the bits must match);
  * against gemm_sm100_tn as it chooses by itself, within the tolerance of the other parity
    tests (max|C - C_ref| / max|C_ref| <= 2e-2 for bf16 output);
  * against the CPU oracle, same tolerance.
"""
import ctypes

import pytest
import torch

from conftest import capi_gemm, capi_status
from oracle import oracle

pytestmark = pytest.mark.gpu


def call_static(capi, A, B, C):
    M, K = A.shape
    N = B.shape[0]
    err = ctypes.c_int(0)
    stream = torch.cuda.current_stream().cuda_stream
    code = {torch.bfloat16: 0, torch.float16: 1}[A.dtype]
    rc = capi.gemm_sm100_tn_static_scratch(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, K, K, N, code,
                                           stream, ctypes.byref(err))
    return rc, err.value


def reset(capi):
    for name, value in ((b"tile_config", -1), (b"split_k", -1), (b"max_ctas", 0), (b"group_m", 0)):
        assert capi.gemm_sm100_set_option(name, value) == 0


def test_static_scratch_matches_workspace_entry_twice_in_a_row(capi):
    reset(capi)
    assert capi.gemm_sm100_static_scratch_capacity() == 5 * 1024 * 1024 + 1024
    # two different problems back to back: the second must not see what the first left behind
    problems = [(16, 28672 // 4, 4096, 90), (32, 1000, 8200, 91)]
    for (M, N, K, seed) in problems:
        A, B = oracle.make_inputs(M, N, K, seed, torch.bfloat16, a_std=1.0, b_std=0.02)
        Ad, Bd = A.cuda(), B.cuda()
        C_static = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc, cuda_err = call_static(capi, Ad, Bd, C_static)
        assert (rc, cuda_err) == (0, 0)
        assert capi_status(capi) == (0, 0)

        # existing entry point, same kernel and schedule, scratch from the caller
        capi.gemm_sm100_set_option(b"tile_config", 2)
        capi.gemm_sm100_set_option(b"split_k", 1)
        C_same = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert capi_gemm(capi, Ad, Bd, C_same) == 0
        reset(capi)
        # existing entry point, its own choice of kernel
        C_auto = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert capi_gemm(capi, Ad, Bd, C_auto) == 0
        assert capi_status(capi) == (0, 0)

        got = C_static.cpu()
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got.view(torch.int16), C_same.cpu().view(torch.int16))
        assert oracle.normalized_max_error(got, C_auto.cpu().float()) <= oracle.tolerance(torch.bfloat16)
        assert oracle.normalized_max_error(got, oracle.reference_matmul_fp32(A, B)) <= oracle.tolerance(torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_static_scratch_same_problem_twice_and_fp16(capi, dtype):
    """The same problem twice in a row on the shared array (the second call finds the first call's
    counters and partial tiles in it and must not be fooled by them), in both element types:
    both results equal, bit for bit, the workspace entry point forced onto the same schedule."""
    reset(capi)
    M, N, K = 24, 3000 + 8, 4096 + 64
    A, B = oracle.make_inputs(M, N, K, 92, dtype, a_std=1.0, b_std=0.02)
    Ad, Bd = A.cuda(), B.cuda()
    capi.gemm_sm100_set_option(b"tile_config", 2)
    capi.gemm_sm100_set_option(b"split_k", 1)
    C_same = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    assert capi_gemm(capi, Ad, Bd, C_same) == 0
    reset(capi)
    assert capi_status(capi) == (0, 0)
    want = C_same.cpu()
    assert oracle.normalized_max_error(want, oracle.reference_matmul_fp32(A, B)) <= oracle.tolerance(dtype)
    for _ in range(2):
        C_static = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
        assert call_static(capi, Ad, Bd, C_static) == (0, 0)
        assert capi_status(capi) == (0, 0)
        assert torch.equal(C_static.cpu().view(torch.int16), want.view(torch.int16))


def test_static_scratch_refuses_what_does_not_fit(capi):
    reset(capi)
    M, N, K = 64, 28672, 8192        # 148 partial tiles of 64 x 256 floats = 9.25 MiB > 5 MiB
    A = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((N, K), dtype=torch.bfloat16, device="cuda")
    C = torch.full((M, N), 7.0, dtype=torch.bfloat16, device="cuda")
    rc, cuda_err = call_static(capi, A, B, C)
    assert rc == 10 and cuda_err == 0            # GEMM_SM100_ERR_STATIC_SCRATCH
    assert b"scratch" in capi.gemm_sm100_error_string(rc)
    torch.cuda.synchronize()
    assert torch.all(C == 7.0)                   # nothing was launched
    # the same problem on a small grid fits (one partial tile per CTA)
    capi.gemm_sm100_set_option(b"max_ctas", 64)
    rc, cuda_err = call_static(capi, A, B, C)
    reset(capi)
    assert (rc, cuda_err) == (0, 0)
    assert capi_status(capi) == (0, 0)
    assert torch.all(C == 0.0)
