"""Per-shape benchmark table: gemm_tn_test vs torch.mm (cuBLAS) on the same GPU.

Successor of the part of the reference's kernels/tests/gemm_bench.py that times its own kernel
and torch.mm (benchmark_gemm_custom :278-295, benchmark_comparison :451-585,
profile_different_shapes :610-706).  Differences: CUDA-event timing on the stream instead of
perf_counter around a synchronised call, the two implementations timed in alternation (10 warm-up
and 30 timed iterations each; the speed-up is the median of the per-iteration ratios), operands
created once per shape, L2 flushed between iterations by writing a 512 MiB scratch buffer (the reference allocates an 80 MB tensor per run,
:58-61), a B200 entry in the peak table (:592-599 has none), and one JSON line per shape.
Its ctypes-cuBLAS autotuner (:124-276) is not reproduced.

A/B mode (the tables under profiles/ that compare tile configurations and K-split schedules come
from it): `--ab` takes variants as `name:option=value,option=value;...` (options of
gemm_kernels.set_option; `auto` = the library's own choice, `mm` = torch.mm), `--shapes` a list of
MxNxK.  The variants are timed in alternation in one process, `--rounds` rounds of `--iters`
back-to-back launches each (or, with `--flush`, single launches with an L2 flush before each),
CUDA events; the table gives the median time per launch and the median per-round ratio to the first
variant.  Under the power cap the clock drifts within seconds, so only numbers from one run of this
mode are comparable.

    python cute-examples_b200/tests/gemm_bench.py --shapes 4096x4096x4096,8192x8192x8192 \
        --ab "c0:tile_config=0;c1:tile_config=1;c8:tile_config=8;auto;mm" --flush
    python cute-examples_b200/tests/gemm_bench.py --ksplit-table
    python cute-examples_b200/tests/gemm_bench.py --fanout 1,4,8 --shapes 8192x4096x8192
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


OPTION_DEFAULTS = {"tile_config": -1, "split_k": -1, "group_m": 0, "k_rotate": -1, "max_ctas": 0, "balance": 1, "tiles_n": 0, "pdl": 1, "early_prefetch": 1, "sk_cluster": -1}

KSPLIT_SHAPES = ("512x4096x4096,1024x4096x4096,256x8192x8192,256x512x65536,512x512x32768,1024x1024x16384,"
                 "2048x2048x8192,1024x2048x8192,512x4096x8192,128x2048x16384,256x256x32768,1024x1024x4096,"
                 "2048x1024x4096,512x1024x65536")
KSPLIT_VARIANTS = ("c0:tile_config=0,split_k=0;c3:tile_config=3,split_k=0;c2s:tile_config=2,split_k=1;"
                   "c0e2:tile_config=0,split_k=2,sk_cluster=0;c0e4:tile_config=0,split_k=4,sk_cluster=0;"
                   "c0e8:tile_config=0,split_k=8;c0e16:tile_config=0,split_k=16;"
                   "c2e2:tile_config=2,split_k=2,sk_cluster=0;c2e4:tile_config=2,split_k=4,sk_cluster=0;"
                   "c2e8:tile_config=2,split_k=8;c2e16:tile_config=2,split_k=16;"
                   "c0k2:tile_config=0,split_k=2,sk_cluster=1;c0k4:tile_config=0,split_k=4,sk_cluster=1;"
                   "c2k2:tile_config=2,split_k=2,sk_cluster=1;c2k4:tile_config=2,split_k=4,sk_cluster=1;"
                   "c11:tile_config=11,split_k=0;c11k2:tile_config=11,split_k=2,sk_cluster=1;"
                   "c11e4:tile_config=11,split_k=4;c11e8:tile_config=11,split_k=8;auto;mm")


def parse_variants(text):
    out = []
    for item in text.split(";"):
        item = item.strip()
        if not item:
            continue
        name, _, opts = item.partition(":")
        settings = {}
        for kv in opts.split(","):
            if kv.strip():
                k, v = kv.split("=")
                settings[k.strip()] = int(v)
        out.append((name.strip(), settings))
    return out


def apply_options(settings):
    for k, v in OPTION_DEFAULTS.items():
        gk.set_option(k, settings.get(k, v))


def timed(fn, iters, scratch=None, cooldown=0.0):
    """µs per call: `iters` back-to-back calls between two events (after `cooldown` seconds of idle
    GPU, if given: a short burst then runs before the power cap reacts, as the first steps of a
    benchmark do), or (with a scratch buffer) single calls with an L2 flush before each, median."""
    if cooldown > 0.0:
        import time

        torch.cuda.synchronize()
        time.sleep(cooldown)
        fn()                                  # clocks up, instruction cache warm
    if scratch is None:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        e.synchronize()
        return s.elapsed_time(e) / iters * 1e3
    times = []
    for _ in range(iters):
        scratch.add_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e) * 1e3)
    return statistics.median(times)


def ab_table(shapes, variants, dtype, rounds, iters, scratch, fanout=None, cooldown=0.0):
    """Interleaved timing of option variants (and torch.mm) per shape; one JSON line per shape."""
    for (M, N, K) in shapes:
        A = (torch.randn((M, K), device="cuda") / K ** 0.5).to(dtype)
        B = (torch.randn((N, K), device="cuda") / K ** 0.5).to(dtype)
        C = torch.empty((M, N), device="cuda", dtype=dtype)
        n_iters = iters if iters > 0 else max(5, min(50, int(20e-3 / (2.0 * M * N * K / 1.4e15 + 8e-6))))
        calls = {}
        outs = None
        if fanout:
            outs = [torch.empty((M, N), device="cuda", dtype=dtype) for _ in range(max(fanout))]
        for name, settings in variants:
            if name == "mm":
                calls[name] = (settings, lambda: torch.mm(A, B.T, out=C))
            elif fanout:
                for n_out in fanout:
                    ptrs = [o.data_ptr() for o in outs[:n_out]]
                    calls[f"{name}/out{n_out}"] = (settings, lambda ptrs=ptrs: gk.gemm_tn_fanout(A, B, ptrs, N))
            else:
                calls[name] = (settings, lambda: gk.gemm_tn_test(A, B, C))
        res = {k: [] for k in calls}
        for k, (settings, fn) in calls.items():
            apply_options(settings)
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        order = list(calls.items())
        for r in range(rounds):
            # every round starts at another variant: what a variant inherits from its predecessor
            # (clock state, L2 contents) then averages out instead of sticking to one of them
            for k, (settings, fn) in order[r % len(order):] + order[:r % len(order)]:
                apply_options(settings)
                res[k].append(timed(fn, n_iters, scratch, cooldown))
        apply_options({})
        gk.device_status()
        first = next(iter(res))
        rec = {"M": M, "N": N, "K": K, "dtype": str(dtype).replace("torch.", ""), "rounds": rounds, "iters": n_iters,
               "flush": scratch is not None, "cooldown_s": cooldown,
               "auto": gk.describe_config(gk.select_config(M, N, K, gk.DTYPE_CODES[dtype])),
               "auto_workspace_bytes": gk.workspace_bytes(M, N, K, gk.DTYPE_CODES[dtype]),
               "auto_plan": gk.describe_plan(M, N, K, gk.DTYPE_CODES[dtype]),
               "us": {k: round(statistics.median(v), 2) for k, v in res.items()},
               "min_us": {k: round(min(v), 2) for k, v in res.items()},
               "ratio_to_first": {k: round(statistics.median(v) / statistics.median(res[first]), 4)
                                  for k, v in res.items()},
               "tflops": {k: round(2.0 * M * N * K / statistics.median(v) / 1e6, 1) for k, v in res.items()},
               "gbs": {k: round(2.0 * (M * K + N * K + M * N) / statistics.median(v) / 1e3, 1) for k, v in res.items()}}
        print(f"{M}x{N}x{K}: " + "  ".join(f"{k} {rec['us'][k]:.1f}us (x{rec['ratio_to_first'][k]:.3f}, min "
                                            f"{rec['min_us'][k]:.1f})" for k in res), flush=True)
        print(json.dumps(rec), flush=True)
        del A, B, C, outs


def sweep(dtype):
    """Grid of shapes (M, N in 128..8192, K in 512..32768, at most 8192^3 flops), the library's own
    plan against cuBLAS (torch.mm) in alternation, three rounds each of back-to-back launches
    (operands stay in L2 where they fit); prints the worst and best ratios, the geometric mean and
    a Markdown table of all shapes by K."""
    import math

    def timed_us(fn, iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        torch.cuda.synchronize()
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) * 1e3 / iters

    dims = [128, 256, 512, 1024, 2048, 4096, 8192]
    rows = []
    for K in (512, 2048, 8192, 32768):
        for M in dims:
            for N in dims:
                if M * N * K > 8192 ** 3 or (K == 32768 and M * N > 2048 * 2048):
                    continue
                A = (torch.randn(M, K, device="cuda") / K ** 0.5).to(dtype)
                B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(dtype)
                C, C2 = torch.empty(M, N, dtype=dtype, device="cuda"), torch.empty(M, N, dtype=dtype, device="cuda")
                iters = max(5, min(100, int(2e4 / max(1.0, 2.0 * M * N * K / 1.2e9))))
                ours, mm = [], []
                for _ in range(3):
                    ours.append(timed_us(lambda: gk.gemm_tn_test(A, B, C), iters))
                    mm.append(timed_us(lambda: torch.mm(A, B.T, out=C2), iters))
                o, m = statistics.median(ours), statistics.median(mm)
                rows.append((o / m, M, N, K, o, m, gk.describe_plan(M, N, K, 0 if dtype == torch.bfloat16 else 1)))
                del A, B, C, C2
    gk.device_status()
    ranked = sorted(rows, reverse=True)
    print("ours / cuBLAS time, worst 15:")
    for r in ranked[:15]:
        print(f"  {r[0]:.2f}  {r[1]}x{r[2]}x{r[3]}  ours {r[4]:.1f} us  cuBLAS {r[5]:.1f} us  | {r[6].split(';')[0]};{r[6].split(';')[1]}")
    print("best 8:")
    for r in ranked[-8:]:
        print(f"  {r[0]:.2f}  {r[1]}x{r[2]}x{r[3]}  ours {r[4]:.1f} us  cuBLAS {r[5]:.1f} us")
    print(f"geometric mean of ours / cuBLAS over {len(rows)} shapes: {math.exp(sum(math.log(r[0]) for r in rows) / len(rows)):.3f}")
    for K in (512, 2048, 8192, 32768):
        sub = {(r[1], r[2]): r[0] for r in rows if r[3] == K}
        if not sub:
            continue
        print(f"\nK = {K}: ours / cuBLAS time (rows M, columns N)\n")
        print("| M \\ N | " + " | ".join(str(n) for n in dims) + " |")
        print("|---|" + "---|" * len(dims))
        for M in dims:
            print(f"| {M} | " + " | ".join(f"{sub[(M, N)]:.2f}" if (M, N) in sub else "" for N in dims) + " |")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--quick", action="store_true", help="skip the largest shapes")
    ap.add_argument("--layout", default="tn", choices=["tn", "nn"], help="B as [N,K] (tn) or as [K,N] (nn)")
    ap.add_argument("--ab", default=None, help="A/B mode: variants 'name:opt=val,...;name2:...;auto;mm'")
    ap.add_argument("--shapes", default=None, help="A/B mode: comma-separated MxNxK")
    ap.add_argument("--rounds", type=int, default=6)
    ap.add_argument("--iters", type=int, default=0, help="launches per round (0 = about 20 ms worth)")
    ap.add_argument("--flush", action="store_true", help="A/B mode: single launches with an L2 flush before each")
    ap.add_argument("--cooldown", type=float, default=0.0,
                    help="A/B mode: idle seconds before every measurement (burst regime instead of the power-capped one)")
    ap.add_argument("--ksplit-table", action="store_true", help="A/B mode preset: K-split schedules on few-tile problems")
    ap.add_argument("--fanout", default=None, help="A/B mode on gemm_tn_fanout with these output counts (local buffers)")
    ap.add_argument("--sweep", action="store_true", help="grid of shapes against cuBLAS, worst / best ratios and geometric mean")
    args = ap.parse_args()
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    if args.sweep:
        print(f"device: {torch.cuda.get_device_name()}  SMs: {gk.num_sms()}")
        sweep(dtype)
        return
    if args.ksplit_table:
        args.ab = args.ab or KSPLIT_VARIANTS
        args.shapes = args.shapes or KSPLIT_SHAPES
        args.iters = args.iters or 50
    if args.ab or args.fanout:
        shapes = [tuple(int(x) for x in sh.split("x")) for sh in (args.shapes or "8192x8192x8192").split(",")]
        variants = parse_variants(args.ab or "auto")
        scratch = torch.zeros(512 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda") if args.flush else None
        fanout = [int(x) for x in args.fanout.split(",")] if args.fanout else None
        print(f"device: {torch.cuda.get_device_name()}  SMs: {gk.num_sms()}")
        ab_table(shapes, variants, dtype, args.rounds, args.iters, scratch, fanout, args.cooldown)
        return
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
