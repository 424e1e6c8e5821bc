"""Per-role stall breakdown of one launch, from the kernel's own trace counters.

Complements profiler.py (a bare launch for Nsight): registers a trace buffer
(gemm_kernels.set_trace_buffer), launches gemm_tn_test once per configuration and prints, for
the leader CTAs, how the MMA issue loop compares with the ideal tensor time, how long each role
waited, and the SM clock during the launch.  `--experiments` also runs the diagnostic variants
"no loads" (pure MMA issue/execute rate) and "no MMA" (pure load rate); their results are garbage
by design.  The reference has no counterpart (its only profiling hook is
kernels/tests/profiler.py:1-12).

    python cute-examples_b200/tests/trace_report.py --m 8192 --n 8192 --k 8192 --configs 0,1,2 --experiments
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import numpy as np  # noqa: E402
import torch  # noqa: E402

import gemm_kernels as gk  # noqa: E402

WORDS = 16
(ENTRY, SETUP, MMA_FIRST, MMA_STALL_FULL, MMA_STALL_ACC, MMA_END, PROD_STALL, PROD_END, EPI_STALL, EPI_END,
 EXIT, TILES, T0_NS, T1_NS) = range(14)


def describe(index):
    text = gk.describe_config(index)
    fields = dict(f.split("=") for f in text.split())
    tile_n = int(fields["tile"].split("x")[1])
    return text, int(fields["cta_group"]), tile_n


FANOUT = 0   # > 0: trace the store-to-every-output kernel with this many outputs (all in local memory)


def run(M, N, K, config, flags, warm=3):
    A = (torch.randn(M, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    B = (torch.randn(N, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
    C = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    gk.set_option("tile_config", config)
    gk.set_option("balance", 0)              # uniform tiles: the ideal cycle count below assumes them
    gk.set_option("split_k", 0)              # whole tiles: the K-split kernels through the workspace keep no trace
    gk.set_option("debug_flags", flags)
    trace = torch.zeros(gk.num_sms() * WORDS, dtype=torch.int64, device="cuda")
    if FANOUT > 0:
        outs = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(FANOUT)]
        ptrs = [o.data_ptr() for o in outs]
        launch = lambda: gk.gemm_tn_fanout(A, B, ptrs, N)  # noqa: E731
    else:
        launch = lambda: gk.gemm_tn_test(A, B, C)  # noqa: E731
    try:
        for _ in range(warm):
            launch()
        gk.set_trace_buffer(trace)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        launch()
        end.record()
        torch.cuda.synchronize()
    finally:
        gk.set_trace_buffer(None)
        gk.set_option("debug_flags", 0)
        gk.set_option("tile_config", -1)
        gk.set_option("balance", 1)
        gk.set_option("split_k", -1)
    gk.device_status()
    return trace.cpu().numpy().reshape(-1, WORDS).astype(np.float64), start.elapsed_time(end)


def report(M, N, K, config, flags):
    text, group, tile_n = describe(config)
    t, ms = run(M, N, K, config, flags)
    used = t[:, T1_NS] > t[:, T0_NS]
    t = t[used]
    lead = t[::group]                                     # leader CTAs hold the MMA counters
    k_blocks = -(-K // 64)
    ideal = lead[:, TILES] * k_blocks * 4 * (tile_n // 2)   # 128 x tile_n x 16 per MMA = tile_n / 2 cycles
    loop_start = lead[:, MMA_FIRST] if not (flags & 1) else lead[:, SETUP]
    loop = lead[:, MMA_END] - loop_start
    clock = ((t[:, EXIT] - t[:, ENTRY]) / (t[:, T1_NS] - t[:, T0_NS])).mean()
    name = {0: "normal", 1: "no loads", 2: "no stores", 4: "no MMA", 3: "no loads, no stores"}.get(flags, str(flags))
    if FANOUT:
        name += f", {FANOUT} outputs"
    print(f"[{text}] {name}: {ms * 1e3:.1f} us, {2.0 * M * N * K / ms / 1e9:.0f} TFLOP/s-equivalent, SM clock {clock:.3f} GHz")
    print(f"    CTAs {len(t)}, tiles per leader {lead[:, TILES].min():.0f}..{lead[:, TILES].max():.0f}; "
          f"set-up {np.mean(t[:, SETUP] - t[:, ENTRY]):.0f} cycles; first operand stage {np.mean(lead[:, MMA_FIRST] - lead[:, ENTRY]):.0f} cycles after entry")
    print(f"    ideal tensor cycles / MMA loop cycles = {ideal.mean() / loop.mean():.3f} "
          f"(loop {loop.mean():.0f} cycles, whole kernel {np.mean(t[:, EXIT] - t[:, ENTRY]):.0f})")
    # phases in microseconds of this launch's own clock, and how far apart the CTAs start and finish
    us = lambda cycles: cycles / clock / 1e3  # noqa: E731
    span = t[:, T1_NS].max() - t[:, T0_NS].min()
    loops = lead[:, MMA_END] - lead[:, MMA_FIRST]
    print(f"    phases: entry -> first operand stage {us(np.mean(lead[:, MMA_FIRST] - lead[:, ENTRY])):.2f} us, MMA loop "
          f"{us(loops.mean()):.2f} us (fastest CTA {us(loops.min()):.2f}, slowest {us(loops.max()):.2f}), last MMA -> exit "
          f"{us(np.mean(lead[:, EXIT] - lead[:, MMA_END])):.2f} us; first entry -> last exit {span / 1e3:.1f} us; CTAs enter within "
          f"{(t[:, T0_NS].max() - t[:, T0_NS].min()) / 1e3:.1f} us and exit within {(t[:, T1_NS].max() - t[:, T1_NS].min()) / 1e3:.1f} us")
    operand_bytes = 2.0 * (M * K + N * K)
    print(f"    operand bytes / mean MMA loop time = {operand_bytes / (us(loops.mean()) * 1e-6) / 1e12:.2f} TB/s; "
          f"/ first entry -> last exit = {operand_bytes / (span * 1e-9) / 1e12:.2f} TB/s (meaningful for memory-bound shapes)")
    print(f"    waits: MMA on operands {100 * (lead[:, MMA_STALL_FULL] / loop).mean():.1f} %, MMA on a free accumulator "
          f"{100 * (lead[:, MMA_STALL_ACC] / loop).mean():.1f} %, producer on free slots "
          f"{100 * (t[:, PROD_STALL] / np.maximum(1, t[:, PROD_END] - t[:, SETUP])).mean():.1f} %, epilogue on accumulators "
          f"{100 * (t[:, EPI_STALL] / np.maximum(1, t[:, EPI_END] - t[:, SETUP])).mean():.1f} %; "
          f"last MMA issued -> exit {np.mean(lead[:, EXIT] - lead[:, MMA_END]):.0f} cycles")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--configs", default="1")
    ap.add_argument("--experiments", action="store_true")
    ap.add_argument("--max-ctas", type=int, default=0, help="cap the grid (0 = all SMs): per-SM limits without power capping")
    ap.add_argument("--fanout", type=int, default=0,
                    help="trace gemm_tn_fanout with this many outputs in local memory (pair-tile configurations 0 and 1)")
    args = ap.parse_args()
    global FANOUT
    FANOUT = args.fanout
    gk.set_option("max_ctas", args.max_ctas)
    for config in [int(c) for c in args.configs.split(",")]:
        for flags in ([0, 1, 4] if args.experiments else [0]):
            report(args.m, args.n, args.k, config, flags)
    gk.set_option("max_ctas", 0)


if __name__ == "__main__":
    main()
