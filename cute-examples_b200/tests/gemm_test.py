"""Correctness script with the flow of the reference's kernels/tests/gemm_test.py:13-41:
random bf16 operands, C pre-filled with NaN, fp32 torch.matmul as ground truth,
allclose(atol=1e-2, rtol=1e-2).  Added: seeded inputs, fp16, the normalised max-error metric
(<= 2e-2 bf16, <= 5e-3 fp16), non-square and ragged shapes.  Needs a B200."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from gemm_kernels import device_status, gemm_tn_test  # noqa: E402


def measure_error_stats(pred, label):
    abs_diff = torch.abs(pred - label)
    max_err = abs_diff.max().item()
    avg_err = abs_diff.mean().item()
    assert torch.allclose(pred, label, atol=1e-2, rtol=1e-2), \
        f"Outputs are not close enough: max_err={max_err}, avg_err={avg_err}"
    return max_err, avg_err


if __name__ == "__main__":
    shapes = [(4096, 4096, 4096), (2048, 2048, 2048), (1024, 1024, 1024), (8192, 14336, 4096), (100, 264, 72)]
    tol = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
    for dtype in (torch.bfloat16, torch.float16):
        for (M, N, K) in shapes:
            device = "cuda"
            print(f"Testing GEMM for shape M={M} N={N} K={K} with dtype {dtype} on {device}")
            g = torch.Generator(device=device).manual_seed(M + N + K)
            A = (torch.randn((M, K), device=device, generator=g) / K ** 0.5).to(dtype)
            B = (torch.randn((N, K), device=device, generator=g) / K ** 0.5).to(dtype)
            C_custom = torch.empty((M, N), device=device, dtype=dtype)
            C_custom.fill_(float("NaN"))      # detects elements the kernel never wrote
            gemm_tn_test(A, B, C_custom)
            device_status()
            C_reference = torch.matmul(A.float(), B.float().T)
            max_err, avg_err = measure_error_stats(C_custom.float(), C_reference)
            norm = (C_custom.float() - C_reference).abs().max().item() / C_reference.abs().max().item()
            assert norm <= tol[dtype], f"normalised max error {norm}"
            print(f"Max error: {max_err}, Avg error: {avg_err}, normalised max error: {norm:.3e}")
    print("all shapes passed")
