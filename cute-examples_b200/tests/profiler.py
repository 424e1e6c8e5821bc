"""Profiling target: a few launches of gemm_tn_test (or, with --cublas, of torch.mm on the same
operands, for a like-for-like counter comparison) on one shape, nothing else.

Successor of the reference's kernels/tests/profiler.py:1-12 (one 4096 x 4096 launch meant to be
run under Nsight).  tests/ncu_capture.py runs it under `ncu --clock-control none -k regex:gemm_tn ...`
and prints the counter table.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402

from gemm_kernels import device_status, gemm_tn_test, set_option  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--m", type=int, default=4096)
ap.add_argument("--n", type=int, default=4096)
ap.add_argument("--k", type=int, default=4096)
ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
ap.add_argument("--launches", type=int, default=3)
ap.add_argument("--tile-config", type=int, default=-1)
ap.add_argument("--option", action="append", default=[], help="name=value for gemm_kernels.set_option")
ap.add_argument("--cublas", action="store_true", help="launch torch.mm(A, B.T) instead of this library's kernel")
args = ap.parse_args()

dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
device = "cuda"
set_option("tile_config", args.tile_config)
for item in args.option:
    name, value = item.split("=")
    set_option(name, int(value))
A = (torch.randn((args.m, args.k), device=device) / args.k ** 0.5).to(dtype)
B = (torch.randn((args.n, args.k), device=device) / args.k ** 0.5).to(dtype)
C_custom = torch.empty((args.m, args.n), device=device, dtype=dtype)
for _ in range(args.launches):
    if args.cublas:
        torch.mm(A, B.T, out=C_custom)
    else:
        gemm_tn_test(A, B, C_custom)
device_status()
print("done", args.m, args.n, args.k, args.dtype)
