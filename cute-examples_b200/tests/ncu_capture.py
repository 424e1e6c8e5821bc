"""Scripted Nsight Compute capture of the GEMM kernel for one shape, with the summary table.

Successor of the reference's kernels/tests/profiler.py:1-12 (a bare launch that the user wraps in
Nsight by hand).  For a shape (or a named benchmark configuration) this script

  1. runs the profiling target (tests/profiler.py) plainly and requires exit code 0,
  2. runs it again under `ncu` with the capture rules this project uses on shared GPUs:
     `--clock-control none` always (ncu would otherwise lock the clocks), ONE kernel by name
     (`-k regex:`), two launches (`-c 2`) after one skipped (`-s 1`), a device footprint of a few
     GB at most (refused otherwise), either `--set full` or a short metric list,
  3. converts the report to CSV (`ncu -i ... --page raw --csv`) and prints a Markdown table of the
     counters the tile and stage choices are argued from: duration, SM clock, tensor-pipe
     activity, DRAM bytes (read, write, per launch), DRAM and L2 throughput, L2 hit rate, stall
     reasons, registers, grid.

Raw output goes to `--out` (default profile_out/); only the printed table is meant to be kept.

    python cute-examples_b200/tests/ncu_capture.py --config cfg2-8192
    python cute-examples_b200/tests/ncu_capture.py --m 4096 --n 4096 --k 4096 --tile-config 8 --metrics short
    python cute-examples_b200/tests/ncu_capture.py --summarize profile_out/prof_8192x8192x8192_bf16.csv
"""
import argparse
import csv
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
PROFILER = os.path.join(HERE, "profiler.py")

# Benchmark configurations by name: (M, N, K, dtype)
CONFIGS = {
    "cfg1-1024": (1024, 1024, 1024, "bf16"),
    "cfg2-4096": (4096, 4096, 4096, "bf16"),
    "cfg2-4096-fp16": (4096, 4096, 4096, "fp16"),
    "cfg2-8192": (8192, 8192, 8192, "bf16"),
    "cfg2-8192-fp16": (8192, 8192, 8192, "fp16"),
    "cfg3-up": (8192, 14336, 4096, "bf16"),
    "cfg3-down": (8192, 4096, 14336, "bf16"),
    "cfg4-16": (16, 28672, 8192, "bf16"),
    "cfg4-64": (64, 28672, 8192, "bf16"),
    "cfg4-128": (128, 28672, 8192, "bf16"),
}

SHORT_METRICS = [
    "gpu__time_duration.sum", "sm__cycles_elapsed.avg.per_second", "sm__cycles_active.avg", "sm__cycles_elapsed.avg",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "dram__bytes_read.sum", "dram__bytes_write.sum", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "lts__t_sector_hit_rate.pct", "lts__throughput.avg.pct_of_peak_sustained_elapsed",
    "launch__registers_per_thread", "launch__grid_size",
]

TABLE = [
    ("gpu__time_duration.sum", "duration"),
    ("sm__cycles_elapsed.avg.per_second", "SM clock during capture"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active", "tensor pipe, % of peak (active cycles)"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "tensor pipe, % of peak (elapsed cycles)"),
    ("sm__cycles_active.avg", "sm__cycles_active.avg"),
    ("sm__cycles_elapsed.avg", "sm__cycles_elapsed.avg"),
    ("dram__bytes_read.sum", "dram__bytes_read.sum"),
    ("dram__bytes_write.sum", "dram__bytes_write.sum"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("dram__cycles_active.avg", "dram__cycles_active.avg"),
    ("lts__t_sector_hit_rate.pct", "L2 sector hit rate, %"),
    ("lts__throughput.avg.pct_of_peak_sustained_elapsed", "L2 throughput, % of peak"),
    ("l1tex__throughput.avg.pct_of_peak_sustained_elapsed", "L1/TEX throughput, % of peak"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active, % of peak"),
    ("smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio", "stall long_scoreboard per issue"),
    ("smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio", "stall barrier per issue"),
    ("smsp__average_warps_issue_stalled_wait_per_issue_active.ratio", "stall wait per issue"),
    ("launch__registers_per_thread", "registers per thread"),
    ("launch__shared_mem_per_block_dynamic", "dynamic shared memory per block"),
    ("launch__grid_size", "grid size"),
    ("launch__cluster_size", "cluster size"),
]


def to_bytes(value, unit):
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}.get(unit.strip(), None)
    try:
        return float(value.replace(",", "")) * scale if scale else None
    except ValueError:
        return None


def summarize(csv_path, header=""):
    """Markdown table of the selected counters, one column per captured launch; returns the text."""
    with open(csv_path, newline="") as fh:
        rows = [r for r in csv.reader(fh) if r]
    # the raw page starts with the header row, then a units row, then one row per launch
    start = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    hdr, units, data = rows[start], rows[start + 1], rows[start + 2:]
    lines = []
    if header:
        lines.append(header)
    name_col = hdr.index("Kernel Name")
    lines.append(f"kernel: `{data[0][name_col]}`" if data else "no launches captured")
    lines.append("")
    lines.append("| metric | " + " | ".join(f"launch {i + 1}" for i in range(len(data))) + " |")
    lines.append("|---|" + "---|" * len(data))
    traffic = [0.0] * len(data)
    have_traffic = False
    for key, label in TABLE:
        if key not in hdr:
            continue
        i = hdr.index(key)
        cells = [f"{d[i]} {units[i]}".strip() for d in data]
        lines.append(f"| {label} | " + " | ".join(cells) + " |")
        if key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
            for j, d in enumerate(data):
                b = to_bytes(d[i], units[i])
                if b is not None:
                    traffic[j] += b
                    have_traffic = True
    if have_traffic:
        lines.append("| **traffic** (read + write, per launch) | " + " | ".join(f"{t / 1e6:.1f} MB" for t in traffic) + " |")
    text = "\n".join(lines)
    print(text)
    return text


def run(cmd, log_path=None, limit_s=600):
    print("$ " + " ".join(cmd), flush=True)
    t0 = time.time()
    if log_path:
        with open(log_path, "w") as fh:
            rc = subprocess.run(cmd, stdout=fh, stderr=subprocess.STDOUT, timeout=limit_s).returncode
    else:
        rc = subprocess.run(cmd, timeout=limit_s).returncode
    print(f"  -> exit {rc} after {time.time() - t0:.1f} s", flush=True)
    return rc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=sorted(CONFIGS), default=None, help="a named benchmark configuration")
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--tile-config", type=int, default=-1)
    ap.add_argument("--option", action="append", default=[], help="name=value passed to the target's set_option")
    ap.add_argument("--metrics", default="full", choices=["full", "short"],
                    help="full = --set full (about 40 passes per launch); short = a dozen metrics (a few passes)")
    ap.add_argument("--kernel", default="gemm_tn", help="regex of the kernel name to capture")
    ap.add_argument("--cublas", action="store_true",
                    help="capture cuBLAS (torch.mm) on the same operands instead; --kernel then defaults to its GEMM kernels")
    ap.add_argument("--out", default="profile_out")
    ap.add_argument("--summarize", default=None, help="only print the table of an existing raw CSV")
    args = ap.parse_args()

    if args.summarize:
        summarize(args.summarize)
        return 0
    if args.config:
        M, N, K, dtype = CONFIGS[args.config]
    else:
        if None in (args.m, args.n, args.k):
            ap.error("give --config or --m/--n/--k")
        M, N, K, dtype = args.m, args.n, args.k, args.dtype
    footprint = 2.0 * (M * K + N * K + M * N)
    if footprint > 4e9:
        print(f"refused: operands take {footprint / 1e9:.1f} GB on the device; captures stay below 4 GB "
              f"(ncu saves and restores device memory around every pass)", file=sys.stderr)
        return 2
    ncu = shutil.which("ncu") or "/usr/local/cuda/bin/ncu"
    os.makedirs(args.out, exist_ok=True)
    tag = f"{M}x{N}x{K}_{dtype}" + (f"_cfg{args.tile_config}" if args.tile_config >= 0 else "") + \
          "".join("_" + o.replace("=", "") for o in args.option)
    target = [sys.executable, PROFILER, "--m", str(M), "--n", str(N), "--k", str(K), "--dtype", dtype,
              "--launches", "3", "--tile-config", str(args.tile_config)]
    for o in args.option:
        target += ["--option", o]
    if args.cublas:
        target.append("--cublas")
        tag += "_cublas"
        if args.kernel == "gemm_tn":
            args.kernel = "nvjet|gemm|cutlass"

    # 1. the plain run must succeed before anything is profiled
    if run(target, os.path.join(args.out, f"plain_{tag}.log")) != 0:
        print("not profiled: the plain run failed (see the log)", file=sys.stderr)
        return 1
    # 2. capture: one kernel, launches 2 and 3, clocks left alone
    rep = os.path.join(args.out, f"prof_{tag}")
    cmd = [ncu, "--clock-control", "none", "-k", f"regex:{args.kernel}", "-s", "1", "-c", "2", "-f", "-o", rep]
    cmd += ["--set", "full"] if args.metrics == "full" else ["--metrics", ",".join(SHORT_METRICS)]
    rc = run(cmd + target, os.path.join(args.out, f"ncu_{tag}.log"), limit_s=900)
    if rc != 0:
        print("ncu failed (see the log)", file=sys.stderr)
        return rc
    # 3. raw CSV + table
    raw = os.path.join(args.out, f"prof_{tag}.csv")
    with open(raw, "w") as fh:
        rc = subprocess.run([ncu, "-i", rep + ".ncu-rep", "--page", "raw", "--csv"], stdout=fh).returncode
    if rc != 0:
        return rc
    header = (f"# {M}x{N}x{K} {dtype}, tile_config {args.tile_config}, options {args.option or 'none'}\n\n"
              f"Command: `python cute-examples_b200/tests/ncu_capture.py " + " ".join(sys.argv[1:]) + "`\n"
              f"(ncu --clock-control none -k regex:{args.kernel} -s 1 -c 2, "
              f"{'--set full' if args.metrics == 'full' else 'short metric list'}; device footprint "
              f"{footprint / 1e6:.0f} MB; the plain run exited 0 directly before)\n")
    text = summarize(raw, header)
    with open(os.path.join(args.out, f"summary_{tag}.md"), "w") as fh:
        fh.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
