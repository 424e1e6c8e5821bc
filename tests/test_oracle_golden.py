"""Pins the CPU oracle (both restatements) against fixtures generated from the reference's own
check (tests/golden/make_golden.py).  No GPU."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import oracle

DT = {0: torch.bfloat16, 1: torch.float16}


def _case(golden, name):
    M, N, K, seed, code, ternary = (int(x) for x in golden[f"{name}/meta"])
    dtype = DT[code]
    A = torch.from_numpy(golden[f"{name}/A"].view(np.int16)).view(dtype)
    B = torch.from_numpy(golden[f"{name}/B"].view(np.int16)).view(dtype)
    C_ref = torch.from_numpy(golden[f"{name}/C_ref"])
    return M, N, K, seed, dtype, bool(ternary), A, B, C_ref


def test_fixture_lists_cases(golden):
    names = [str(n) for n in golden["names"]]
    assert {"small_bf16", "ragged_bf16", "small_fp16", "ternary_bf16", "ternary_fp16"} <= set(names)


@pytest.mark.parametrize("name", ["small_bf16", "ragged_bf16", "small_fp16", "ternary_bf16", "ternary_fp16"])
def test_oracles_match_reference_ground_truth(golden, name):
    M, N, K, seed, dtype, ternary, A, B, C_ref = _case(golden, name)
    assert A.shape == (M, K) and B.shape == (N, K) and C_ref.shape == (M, N)
    via_torch = oracle.reference_matmul_fp32(A, B)
    via_c = oracle.c_gemm_tn_f32(A, B)
    if ternary:
        # integer-valued sums: every summation order gives the same bits
        assert torch.equal(via_torch, C_ref)
        assert torch.equal(via_c, C_ref)
    else:
        scale = C_ref.abs().max().item()
        assert (via_torch - C_ref).abs().max().item() <= 2e-6 * scale + 1e-7
        assert (via_c - C_ref).abs().max().item() <= 2e-6 * scale + 1e-7
    # the rounded result of the C restatement passes the reference's own check
    rounded = oracle.c_gemm_tn(A, B)
    max_err, avg_err, ok = oracle.measure_error_stats(rounded.float(), C_ref)
    assert ok
    ideal_max, ideal_avg = golden[f"{name}/ideal_err"]
    assert max_err <= ideal_max * 1.01 + 1e-6
    assert oracle.normalized_max_error(rounded, C_ref) <= oracle.tolerance(dtype)


@pytest.mark.parametrize("name", ["small_bf16", "small_fp16", "ternary_bf16"])
def test_inputs_reproduce_from_seed(golden, name):
    M, N, K, seed, dtype, ternary, A, B, _ = _case(golden, name)
    gen = oracle.make_ternary_inputs if ternary else oracle.make_inputs
    A2, B2 = gen(M, N, K, seed, dtype)
    assert torch.equal(A2.view(torch.int16), A.view(torch.int16))
    assert torch.equal(B2.view(torch.int16), B.view(torch.int16))


def test_config1_rows_and_digests(golden):
    A, B = oracle.make_inputs(1024, 1024, 1024, 0, torch.bfloat16)
    dig = [hashlib.sha256(t.contiguous().view(torch.int16).numpy().tobytes()).hexdigest() for t in (A, B)]
    assert dig == [str(d) for d in golden["cfg1/digests"]]
    rows = [int(r) for r in golden["cfg1/rows"]]
    want = torch.from_numpy(golden["cfg1/C_ref_rows"])
    scale = float(golden["cfg1/absmax"][0])
    got_c = oracle.c_gemm_tn_f32(A[rows], B)
    got_t = oracle.reference_matmul_fp32(A, B)[rows]
    assert (got_c - want).abs().max().item() <= 2e-6 * scale
    assert (got_t - want).abs().max().item() <= 2e-6 * scale
    # an ideal kernel (fp32 accumulate, one rounding) sits ~6x inside the bf16 tolerance
    ideal = oracle.c_gemm_tn(A[rows], B)
    assert oracle.normalized_max_error(ideal, want) < 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_c_conversions_match_torch(dtype):
    allbits = torch.arange(-32768, 32768, dtype=torch.int32).to(torch.int16).view(dtype)
    assert torch.equal(oracle.c_widen_16(allbits).view(torch.int32), allbits.float().view(torch.int32))
    g = torch.Generator().manual_seed(3)
    x = torch.randn(200000, generator=g) * (10.0 ** torch.randint(-9, 6, (200000,), generator=g).float())
    x = torch.cat([x, torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 65504.0, 65519.9, 65520.0, 2.0 ** -25,
                                    2.0 ** -24, 1.0 + 2.0 ** -8, 1.0 + 2.0 ** -11, 3.0e38])])
    assert torch.equal(oracle.c_round_to_16(x, dtype).view(torch.int16), x.to(dtype).view(torch.int16))


def test_edge_shapes_cpu():
    A = torch.zeros((0, 64), dtype=torch.bfloat16)
    B = torch.ones((8, 64), dtype=torch.bfloat16)
    assert oracle.c_gemm_tn_f32(A, B).shape == (0, 8)
    A = torch.ones((4, 0), dtype=torch.bfloat16)
    B = torch.ones((8, 0), dtype=torch.bfloat16)
    assert torch.equal(oracle.c_gemm_tn_f32(A, B), torch.zeros(4, 8))
    eye = torch.eye(64, dtype=torch.bfloat16)
    A, _ = oracle.make_inputs(48, 64, 64, 21)
    assert torch.equal(oracle.c_gemm_tn(A, eye).view(torch.int16), A.view(torch.int16))
