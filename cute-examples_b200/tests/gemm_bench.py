"""Per-shape benchmark table: gemm_tn_test vs torch.mm (cuBLAS) on the same GPU.

Successor of the part of the reference's kernels/tests/gemm_bench.py that times its own kernel
and torch.mm (benchmark_gemm_custom :278-295, benchmark_comparison :451-585,
profile_different_shapes :610-706).  Differences: CUDA-event timing on the stream instead of
perf_counter around a synchronised call, the two implementations timed in alternation (10 warm-up
and 30 timed iterations each; the speed-up is the median of the per-iteration ratios), operands
created once per shape, L2 flushed between iterations by writing a 512 MiB scratch buffer (the reference allocates an 80 MB tensor per run,
:58-61), a B200 entry in the peak table (:592-599 has none), and one JSON line per shape.
Its ctypes-cuBLAS autotuner (:124-276) is not reproduced.
"""
import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

import gemm_kernels as gk  # noqa: E402

# Dense 16-bit tensor peaks in TFLOP/s.  B200 nominal is the dense half of NVIDIA's figure.
GPU_PEAK_TFLOPS = {"B200": 2250.0, "H100": 989.0, "A100": 312.0}
B200_HBM_GBS = 8000.0

REFERENCE_SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 16384),
                    (8192, 8192, 8192), (16384, 16384, 4096)]        # (M=N, K) list of gemm_bench.py:616-623
TARGET_SHAPES = [(8192, 14336, 4096), (8192, 4096, 14336), (16, 28672, 8192), (64, 28672, 8192),
                   (128, 28672, 8192)]


def peak_for_device():
    name = torch.cuda.get_device_name()
    for key, val in GPU_PEAK_TFLOPS.items():
        if key in name:
            return key, val
    return name, None


def time_pair(ours, theirs, scratch, warmup=10, iters=30):
    """Times the two callables in alternation (flush, ours, flush, theirs, ...): under the power cap
    the clock drifts within seconds, and timing one after the other would charge the drift to one
    of them.  Returns (median, min) of each and the median of the per-iteration time ratios."""
    for _ in range(warmup):
        ours()
        theirs()
    torch.cuda.synchronize()
    t_ours, t_theirs = [], []
    for _ in range(iters):
        for fn, times in ((ours, t_ours), (theirs, t_theirs)):
            scratch.add_(1)                                 # evict operands from L2
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            times.append(s.elapsed_time(e))
    ratio = statistics.median(b / a for a, b in zip(t_ours, t_theirs))
    return (statistics.median(t_ours), min(t_ours)), (statistics.median(t_theirs), min(t_theirs)), ratio


def bench_shape(M, N, K, dtype, scratch, peak, layout="tn"):
    A = (torch.randn((M, K), device="cuda") / K ** 0.5).to(dtype)
    C = torch.empty((M, N), device="cuda", dtype=dtype)
    C2 = torch.empty((M, N), device="cuda", dtype=dtype)
    if layout == "tn":
        B = (torch.randn((N, K), device="cuda") / K ** 0.5).to(dtype)    # already [N, K]: no transpose copy
        (ours_med, ours_min), (torch_med, torch_min), ratio = time_pair(
            lambda: gk.gemm_tn_test(A, B, C), lambda: torch.mm(A, B.T, out=C2), scratch)
        gk.device_status()
    else:
        B = (torch.randn((K, N), device="cuda") / K ** 0.5).to(dtype)    # [K, N], as torch.mm takes it
        (ours_med, ours_min), (torch_med, torch_min), ratio = time_pair(
            lambda: gk.gemm_nn(A, B, C), lambda: torch.mm(A, B, out=C2), scratch)
        gk.device_status()
    flops = 2.0 * M * N * K
    nbytes = 2.0 * (M * K + N * K + M * N)
    rec = {
        "M": M, "N": N, "K": K, "dtype": str(dtype).replace("torch.", ""), "layout": layout,
        "ours_ms": round(ours_med, 4), "ours_min_ms": round(ours_min, 4), "torch_ms": round(torch_med, 4),
        "ours_tflops": round(flops / ours_med / 1e9, 1), "torch_tflops": round(flops / torch_med / 1e9, 1),
        "torch_min_ms": round(torch_min, 4), "speedup_vs_torch": round(ratio, 3), "ours_gbs": round(nbytes / ours_med / 1e6, 1),
        "tile_config": gk.describe_config(gk.select_config(M, N, K, gk.DTYPE_CODES[dtype])),
        "max_abs_diff_vs_torch": float((C.float() - C2.float()).abs().max().item()),
    }
    if peak:
        rec["pct_of_nominal_peak"] = round(100.0 * rec["ours_tflops"] / peak, 1)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--quick", action="store_true", help="skip the largest shapes")
    ap.add_argument("--layout", default="tn", choices=["tn", "nn"], help="B as [N,K] (tn) or as [K,N] (nn)")
    args = ap.parse_args()
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    name, peak = peak_for_device()
    print(f"device: {torch.cuda.get_device_name()}  SMs: {gk.num_sms()}  nominal dense peak: {peak} TFLOP/s ({name})")
    scratch = torch.zeros(512 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda")
    shapes = REFERENCE_SHAPES + TARGET_SHAPES
    if args.quick:
        shapes = [s for s in shapes if 2.0 * s[0] * s[1] * s[2] < 2.5e12]
    print(f"{'M':>6} {'N':>6} {'K':>6} | {'ours ms':>9} {'TFLOP/s':>8} {'GB/s':>8} | {'torch ms':>9} {'TFLOP/s':>8} | speed-up")
    for (M, N, K) in shapes:
        r = bench_shape(M, N, K, dtype, scratch, peak, args.layout)
        print(f"{M:>6} {N:>6} {K:>6} | {r['ours_ms']:>9.4f} {r['ours_tflops']:>8.1f} {r['ours_gbs']:>8.1f} | "
              f"{r['torch_ms']:>9.4f} {r['torch_tflops']:>8.1f} | {r['speedup_vs_torch']:.3f}x")
        print(json.dumps(r))


if __name__ == "__main__":
    main()
