#!/usr/bin/env python
"""Benchmark of the sm_100a TN GEMM behind gemm_kernels.gemm_tn_test.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one synthetic
batch:
  * N = 1: the square bf16 GEMM M=N=K=8192 (benchmark configuration 2; operands ~N(0,1)/sqrt(K), seed 1).
  * N > 1: the large GEMM M=N=K=32768 (benchmark configuration 5, seed 4) with B sharded by rows over the
    ranks, every rank computing its column slab of C and the slabs assembled on every rank by
    the GEMM epilogue itself (stores to every GPU's C over NVLink; `--nsplit nccl` selects the
    NCCL all-gather path instead): strong scaling, `value` = 2*M*N*K / (max over ranks of the
    step time).
`value` is timed with CUDA events on the launching stream, operands resident in HBM.
`e2e` is the same step through the public Python entry point with pinned HOST operands and a
HOST result: host->device copies of A and B and the device->host copy of C are inside the
timed region.  `roofline` compares the GEMM kernel with the measured cuBLAS bf16 peak of this
pool (a driver-written JSON file beside this script, else the stated fallback).  `cpu_baseline` times the CPU oracle
(the reference's check expression, torch fp32 matmul) on the host cores.

--impl reference: the reference's implementation of this path is sm_90a device code that cannot
run on sm_100 and has no CPU code; its own ground truth, torch.matmul(A.float(), B.float().T)
(kernels/tests/gemm_test.py:36), timed on the host cores on a bounded slab of the same workload,
stands in (cpu_baseline.kind = "port").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
sys.path.insert(0, str(REPO / "cute-examples_b200"))

import torch  # noqa: E402

# DRAM traffic of one launch of the N=1 workload comes from an ncu capture recorded in
# profiles/dram_traffic.json together with the kernel configuration it was taken with; a record
# whose configuration no longer matches what the library selects is reported as stale (null).
TRAFFIC_RECORD = REPO / "profiles" / "dram_traffic.json"

WORKLOAD_SINGLE = "cfg2 square bf16 TN GEMM M=N=K=8192, fp32 accumulate, bf16 out, seed 1"


def workload_multi(world: int) -> str:
    return f"cfg5 bf16 TN GEMM M=N=K=32768, seed 4, B row-sharded over {world} GPUs, C assembled on every GPU"


FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def load_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            if d.get("bf16_tflops") and d.get("hbm_gbs"):
                return d, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def recorded_traffic(key, live_config):
    """(bytes per launch or None, note) from profiles/dram_traffic.json for workload `key`."""
    try:
        rec = json.loads(TRAFFIC_RECORD.read_text())[key]
    except Exception as exc:  # missing file or workload
        return None, f"no ncu record for {key} ({exc.__class__.__name__})"
    if rec.get("tile_config") != live_config:
        return None, (f"stale: {TRAFFIC_RECORD.name} was captured with [{rec.get('tile_config')}], the library now "
                      f"selects [{live_config}]")
    return int(rec["dram_bytes_per_launch"]), rec.get("source", "")


def base_config(gpus):
    """The `config` object both arms print (same keys and values for the same --gpus)."""
    if gpus == 1:
        return {"workload": WORKLOAD_SINGLE, "M": 8192, "N": 8192, "K": 8192,
                "l2": "operands 256 MiB > 126 MB L2 (inputs larger than L2; no flush between steps)"}
    return {"workload": workload_multi(gpus), "M": 32768, "N": 32768, "K": 32768,
            "l2": "operands 2 GiB + 2/G GiB per GPU > 126 MB L2 (inputs larger than L2)"}


def gemm_flops(M, N, K):
    return 2.0 * M * N * K


def gemm_bytes(M, N, K, esize=2):
    """Algorithmic bytes: each operand read once, C written once."""
    return float(esize) * (M * K + N * K + M * N)


# ------------------------------------------------------------------ clocks ---
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the timed
    region runs."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int, period_s: float = 0.005):
        self.samples, self.reasons, self.power = [], set(), []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": round(max(self.power), 1) if self.power else None}


# ------------------------------------------------------------- GPU helpers ---
def device_inputs(M, N, K, seed, dtype, device, a_std=None, b_std=None):
    """Seeded operands of the benchmark distributions, drawn on the device (statistically the
    same as the CPU generator the parity tests use; bench inputs are not compared bitwise)."""
    g = torch.Generator(device=device).manual_seed(seed)
    sa = (1.0 / K ** 0.5) if a_std is None else a_std
    sb = (1.0 / K ** 0.5) if b_std is None else b_std
    A = (torch.randn((M, K), generator=g, device=device, dtype=torch.float32) * sa).to(dtype)
    B = (torch.randn((N, K), generator=g, device=device, dtype=torch.float32) * sb).to(dtype)
    return A, B


def cfg5_operands(device, n=32768, b_rows=None, slab=4096):
    """Benchmark configuration 5 operands, seed 4: A[n,n] then B[n,n] ~ N(0,1)/sqrt(n) from ONE device
    generator, drawn as fp32 slabs of `slab` rows (0.5 GiB of scratch at a time) and cast to bf16.
    Every caller draws the identical sequence; `b_rows = (lo, hi)` keeps only those rows of B, so
    the ranks of a column-sharded run hold row slabs of the same B that one GPU would use."""
    g = torch.Generator(device=device).manual_seed(4)
    lo, hi = (0, n) if b_rows is None else b_rows
    A = torch.empty((n, n), dtype=torch.bfloat16, device=device)
    B = torch.empty((hi - lo, n), dtype=torch.bfloat16, device=device)
    scale = 1.0 / n ** 0.5
    for r0 in range(0, n, slab):
        A[r0:r0 + slab] = (torch.randn((slab, n), generator=g, device=device) * scale).to(torch.bfloat16)
    for r0 in range(0, n, slab):
        draw = torch.randn((slab, n), generator=g, device=device)       # drawn even when not kept: same stream
        a, b = max(r0, lo), min(r0 + slab, hi)
        if a < b:
            B[a - lo:b - lo] = (draw[a - r0:b - r0] * scale).to(torch.bfloat16)
        del draw
    return A, B


def sampled_rows_error(C_rows, A_rows, B):
    """Normalised max error of sampled rows of C against the CPU oracle (the reference's check
    expression) on the same operands; returns (error, rows checked)."""
    from oracle import oracle

    C_ref = oracle.reference_matmul_fp32(A_rows.cpu(), B.cpu())
    return oracle.normalized_max_error(C_rows.cpu(), C_ref), int(A_rows.shape[0])


def cfg5_single_gpu(gk, peaks, device, steps=5, warmup=3, with_cpu=True):
    """Benchmark configuration 5 (M=N=K=32768) on ONE GPU: the strong-scaling baseline of the
    multi-GPU runs, same operands (seed 4), timed back to back (a launch takes about 50 ms, so
    this is the sustained, power-capped regime and the sustained cuBLAS peak is the divisor)."""
    n = 32768
    A, B = cfg5_operands(device, n)
    C = torch.empty((n, n), dtype=torch.bfloat16, device=device)
    for _ in range(warmup):
        gk.gemm_tn_test(A, B, C)
    torch.cuda.synchronize()
    ms = time_steps(lambda: gk.gemm_tn_test(A, B, C), steps, torch.cuda.synchronize) / steps
    gk.device_status()
    tf = gemm_flops(n, n, n) / ms / 1e9
    peak = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
    rec = {"shape": "cfg5 32768^3 bf16 (1 GPU)", "ms": round(ms, 3), "tflops": round(tf, 1),
           "gbs": round(gemm_bytes(n, n, n) / ms / 1e6, 1), "bound": "tensor", "steps": steps, "warmup": warmup,
           "l2": "operands 4 GiB > L2, back to back", "frac": round(tf / peak, 4), "peak": "bf16_tflops_sustained",
           "note": "the same workload the --gpus N runs split over N GPUs: efficiency = value_N / (N x this)"}
    if with_cpu:
        rows = torch.tensor([0, 255, 256, 9999, 16384, 20000, 32767, 12345, 4097, 8191, 30000, 77, 25000, 1, 511, 31999])
        err, count = sampled_rows_error(C[rows.to(device)], A[rows.to(device)], B)
        rec["norm_max_err"] = float(f"{err:.3e}")
        rec["rows_checked"] = count
    del A, B, C
    return rec


def time_steps(fn, steps, sync, barrier=None):
    """Exactly `steps` calls of fn between two events on the current stream; returns ms total."""
    if barrier:
        barrier()
    sync()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    sync()
    if barrier:
        barrier()
    return start.elapsed_time(end)


def flush_l2(buf):
    buf.add_(1)


def cpu_rows_for(M, N, K, target_flops=6.0e10):
    """Rows of A for the CPU leg of a shape: the whole problem when it is small, else a slab worth
    about `target_flops` (a fraction of a second on a server CPU)."""
    rows = int(max(64, min(M, target_flops / (2.0 * N * K))))
    return M if rows >= M else max(64, rows // 64 * 64)


def secondary_shapes(gk, peaks, device, with_cpu=True):
    """Other benchmark shapes, reported beside the headline.  Tensor-bound shapes: L2 flushed
    between iterations by writing a 512 MiB buffer (several of them fit in the 126 MB L2).
    HBM-bound small-M shapes: timed back to back with no flush, because their streamed operand
    (B, 470 MB) is larger than L2 by itself and a flush would leave 126 MB of dirty lines whose
    write-back competes with the very bandwidth being measured."""
    out = []
    scratch = torch.zeros(512 * 1024 * 1024 // 4, dtype=torch.int32, device=device)
    cases = [
        ("cfg1 1024^3 bf16", 1024, 1024, 1024, torch.bfloat16, 0, None, None, "tensor"),
        ("cfg2 4096^3 bf16", 4096, 4096, 4096, torch.bfloat16, 1, None, None, "tensor"),
        ("cfg2 4096^3 fp16", 4096, 4096, 4096, torch.float16, 1, None, None, "tensor"),
        ("cfg2 8192^3 fp16", 8192, 8192, 8192, torch.float16, 1, None, None, "tensor"),
        ("cfg3 8192x14336x4096 bf16", 8192, 14336, 4096, torch.bfloat16, 2, 1.0, 0.02, "tensor"),
        ("cfg3 8192x4096x14336 bf16", 8192, 4096, 14336, torch.bfloat16, 2, 1.0, 0.02, "tensor"),
        ("cfg4 16x28672x8192 bf16", 16, 28672, 8192, torch.bfloat16, 3, 1.0, 0.02, "hbm"),
        ("cfg4 64x28672x8192 bf16", 64, 28672, 8192, torch.bfloat16, 3, 1.0, 0.02, "hbm"),
        ("cfg4 128x28672x8192 bf16", 128, 28672, 8192, torch.bfloat16, 3, 1.0, 0.02, "hbm"),
    ]
    for name, M, N, K, dtype, seed, sa, sb, bound in cases:
        A, B = device_inputs(M, N, K, seed, dtype, device, sa, sb)
        C = torch.empty((M, N), dtype=dtype, device=device)
        for _ in range(3):
            gk.gemm_tn_test(A, B, C)
        torch.cuda.synchronize()
        times = []
        if bound == "hbm":
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(10):
                    gk.gemm_tn_test(A, B, C)
                e.record()
                e.synchronize()
                times.append(s.elapsed_time(e) / 10)
        else:
            for _ in range(10):
                flush_l2(scratch)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                gk.gemm_tn_test(A, B, C)
                e.record()
                e.synchronize()
                times.append(s.elapsed_time(e))
        ms = statistics.median(times)
        ms_b2b = None
        if bound == "tensor" and gemm_bytes(M, N, K) < 120e6:
            # operands fit L2: also the warm figure, 20 launches back to back (launches then overlap
            # with their predecessor's tail, which a flush kernel in between prevents)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(20):
                gk.gemm_tn_test(A, B, C)
            e.record()
            e.synchronize()
            ms_b2b = s.elapsed_time(e) / 20
        tf = gemm_flops(M, N, K) / ms / 1e9
        gbs = gemm_bytes(M, N, K) / ms / 1e6
        rec = {"shape": name, "ms": round(ms, 4), "tflops": round(tf, 1), "gbs": round(gbs, 1), "bound": bound,
               "l2": "inputs larger than L2, back to back" if bound == "hbm" else "flushed between iterations"}
        if ms_b2b is not None:
            rec["ms_back_to_back_warm_l2"] = round(ms_b2b, 4)
            rec["tflops_back_to_back_warm_l2"] = round(gemm_flops(M, N, K) / ms_b2b / 1e9, 1)
        if bound == "tensor":
            rec["frac"] = round(tf / peaks["bf16_tflops"], 4)
        else:
            rec["frac"] = round(gbs / peaks["hbm_gbs"], 4)
        if with_cpu:
            # the same operands on the host cores: the reference's check expression, fp32
            from oracle import oracle

            rows = cpu_rows_for(M, N, K)
            Ac, Bc = A[:rows].cpu(), B.cpu()
            sec, threads, C_ref = oracle.time_cpu_matmul(Ac, Bc, min_seconds=0.0, max_runs=1)
            rec["cpu_tflops"] = round(gemm_flops(rows, N, K) / sec / 1e12, 3)
            rec["cpu_cores"] = threads
            rec["cpu_rows"] = rows
            rec["norm_max_err"] = float(f"{oracle.normalized_max_error(C[:rows].cpu(), C_ref):.3e}")
            del Ac, Bc, C_ref
        out.append(rec)
        del A, B, C
    gk.device_status()
    return out


def cpu_baseline_sample(M, N, K, seed, rows, target_seconds=10.0):
    """Times the CPU oracle on `rows` rows of A against all of B (same distributions)."""
    from oracle import oracle

    A, B = oracle.make_inputs(rows, N, K, seed, torch.bfloat16)
    sec, threads, _ = oracle.time_cpu_matmul(A, B, min_seconds=target_seconds, max_runs=5)
    tf = gemm_flops(rows, N, K) / sec / 1e12
    return {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"torch fp32 matmul (the reference's check expression) of {rows} rows of A "
                      f"x all of B, N={N} K={K}; {sec:.3f} s per call; host has {os.cpu_count()} logical cores"}


# --------------------------------------------------------------- reference ---
def run_reference(args, rank):
    if rank != 0:
        return
    from oracle import oracle

    # All host cores, whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1 for its
    # children, which made this arm 16x slower at N > 1 than at N = 1).
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(cores)
    cfg = base_config(args.gpus)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    seed = 1 if args.gpus == 1 else 4
    rows = 1024 if args.gpus == 1 else 256
    A, B = oracle.make_inputs(rows, N, K, seed, torch.bfloat16)
    for _ in range(min(args.warmup, 2)):
        oracle.reference_matmul_fp32(A, B)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.reference_matmul_fp32(A, B)
    sec = (time.perf_counter() - t0) / args.steps
    tf = gemm_flops(rows, N, K) / sec / 1e12
    sample = (f"each step = torch fp32 matmul of a {rows}-row slab of A x all of B (N={N}, K={K}) on "
              f"{torch.get_num_threads()} threads; TFLOP/s of the slab stands for the whole GEMM")
    line = {
        "impl": "reference", "metric": "bf16 GEMM TFLOP/s", "value": round(tf, 4), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": round(tf, 4), "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": round(tf, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------- ours ---
def run_single(args):
    import gemm_kernels as gk

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    peaks, peak_src = load_peaks()
    M = N = K = 8192
    dtype = torch.bfloat16
    A, B = device_inputs(M, N, K, 1, dtype, device)
    C = torch.empty((M, N), dtype=dtype, device=device)
    step = lambda: gk.gemm_tn_test(A, B, C)  # noqa: E731
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    with ClockSampler(0) as clk:
        ms_total = time_steps(step, args.steps, torch.cuda.synchronize)
    gk.device_status()
    ms = ms_total / args.steps
    tflops = gemm_flops(M, N, K) / ms / 1e9
    # SM cycles one launch needs (from the per-CTA trace counters; independent of the clock):
    # cycles / measured time per step = the clock the timed region really ran at
    traced = gk.trace_launch(A, B, C)
    sm_mhz_effective = traced["cycles"] / (ms * 1e3)

    # end to end through the public host-memory entry point: pinned host operands in, host result
    # out, every step (uploads of A panels, GEMM panels and downloads of C panels overlap)
    Ah, Bh = A.cpu().pin_memory(), B.cpu().pin_memory()
    Ch = torch.empty((M, N), dtype=dtype).pin_memory()
    host_gemm = gk.HostGemm(M, N, K, dtype, device)

    def e2e_step():
        host_gemm(Ah, Bh, Ch)

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = time_steps(e2e_step, e2e_steps, torch.cuda.synchronize) / e2e_steps
    gk.device_status()
    e2e_tflops = gemm_flops(M, N, K) / e2e_ms / 1e9
    e2e_check = float((Ch[::1024].float() - C[::1024].cpu().float()).abs().max().item())

    # what the upload alone costs on this box: the floor of the end-to-end step (the download of C
    # and the GEMMs run under it)
    def upload_only():
        host_gemm.A.copy_(Ah, non_blocking=True)
        host_gemm.B.copy_(Bh, non_blocking=True)

    upload_only()
    torch.cuda.synchronize()
    h2d_floor_ms = time_steps(upload_only, 5, torch.cuda.synchronize) / 5
    del host_gemm

    del A, B, C, Ah, Bh, Ch
    torch.cuda.empty_cache()
    shapes = [] if args.no_shapes else secondary_shapes(gk, peaks, device, with_cpu=not args.no_cpu)
    scaling_baseline = None
    if not args.no_shapes:
        torch.cuda.empty_cache()
        scaling_baseline = cfg5_single_gpu(gk, peaks, device, with_cpu=not args.no_cpu)
        shapes.append(scaling_baseline)
    cpu = None if args.no_cpu else cpu_baseline_sample(M, N, K, 1, rows=2048)
    live_config = gk.describe_config(gk.select_config(M, N, K, 0))
    traffic, traffic_note = recorded_traffic("8192x8192x8192_bf16", live_config)

    timed_s = ms_total / 1e3
    peak_key = "bf16_tflops" if timed_s <= 1.0 else "bf16_tflops_sustained"
    peak = float(peaks.get(peak_key) or peaks["bf16_tflops"])
    line = {
        "metric": "bf16 GEMM TFLOP/s", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": base_config(1),
        "kernel_config": live_config,
        "e2e": {"value": round(e2e_tflops, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "ms_per_step": round(e2e_ms, 4), "steps": e2e_steps,
                "api": "gemm_kernels.HostGemm (A uploaded in row panels; GEMM and download of C per panel)",
                "max_abs_diff_vs_device_path": e2e_check,
                "upload_only_ms": round(h2d_floor_ms, 4),
                "upload_only_note": "the same pinned A and B copied to the device with nothing else running: the floor "
                                    "of the step on this box's PCIe link"},
        "gpu_launches": args.steps,
        "clocks": dict(clk.summary(), kernel_cycles=round(traced["cycles"]),
                       sm_mhz_effective=round(sm_mhz_effective),
                       note="sm_mhz / reasons: NVML samples during the timed region (NVML does not follow the "
                            "fast power-cap steps); kernel_cycles: SM cycles of one launch from the kernel's "
                            "trace counters; sm_mhz_effective = kernel_cycles / ms_per_step"),
        "roofline": {"bound": "tensor", "achieved": round(tflops, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tflops / peak, 4), "traffic": traffic,
                     "traffic_source": traffic_note, "algorithmic_bytes": gemm_bytes(M, N, K),
                     "peak_source": f"{peak_src}:{peak_key}", "kernel": "gemm_sm100::gemm_tn_kernel",
                     "flops_per_launch": gemm_flops(M, N, K)},
        "cpu_baseline": cpu,
        "scaling_baseline": scaling_baseline,
        "shapes": shapes,
    }
    print(json.dumps(line), flush=True)


def c_checksums(C, chunk_rows=2048):
    """Two position-sensitive 64-bit checksums of the bits of C (computed in row chunks so that the
    int64 temporaries stay small): equal on two GPUs only if they hold the same C, bit for bit."""
    M, N = C.shape
    col_w = (torch.arange(N, device=C.device, dtype=torch.int64) % 251) + 1
    plain = torch.zeros((), dtype=torch.int64, device=C.device)
    weighted = torch.zeros((), dtype=torch.int64, device=C.device)
    for r0 in range(0, M, chunk_rows):
        bits = C[r0:r0 + chunk_rows].view(torch.int16).to(torch.int64)
        plain += bits.sum()
        row_w = (torch.arange(r0, r0 + bits.shape[0], device=C.device, dtype=torch.int64) % 241) + 1
        weighted += ((bits * col_w).sum(dim=1) * row_w).sum()
    return torch.stack([plain, weighted])


def run_multi(args):
    import torch.distributed as dist

    import gemm_kernels as gk

    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    peaks, peak_src = load_peaks()
    cfg = base_config(world)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    dtype = torch.bfloat16
    lo, hi = gk.shard_rows(N, world, rank)
    # A (same on every rank) and this rank's rows [lo, hi) of the seed-4 B
    A, B_shard = cfg5_operands(device, N, b_rows=(lo, hi))
    # Default: the all-gather of C folded into the GEMM epilogue (stores to every GPU's C over
    # NVLink, symmetric memory).  --nsplit nccl: per-panel GEMM + NCCL all-gather + re-stride copy.
    mode = args.nsplit
    fused = None
    if mode in ("auto", "fused"):
        try:
            fused = gk.FusedNSplit(M, N, dtype, device)
            mode = "fused"
        except Exception as exc:  # symmetric memory unavailable on this box
            if args.nsplit == "fused":
                raise
            print(f"[bench] symmetric memory unavailable ({exc!r}); using the NCCL all-gather path", file=sys.stderr)
            mode = "nccl"
    if mode == "fused":
        launches_per_step = 1
        step = lambda: fused(A, B_shard)  # noqa: E731
        how = ("all-gather of C fused into the GEMM epilogue (TMA stores to every GPU's C over NVLink), "
               "two alternating C buffers, one cross-GPU barrier per step")
    else:
        C_nccl = torch.empty((M, N), dtype=dtype, device=device)
        plan = gk.NSplitPlan.create(M, N, world, dtype, device, num_panels=args.panels)
        launches_per_step = plan.num_panels
        step = lambda: gk.gemm_tn_nsplit(A, B_shard, C_nccl, plan=plan)  # noqa: E731
        how = f"NCCL all-gather of C, {plan.num_panels} row panels overlapped with the GEMM"

    def barrier():
        dist.barrier(device_ids=[local])

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    with ClockSampler(local) as clk:
        ms_total = time_steps(step, args.steps, torch.cuda.synchronize, barrier)
    gk.device_status()
    t = torch.tensor([ms_total], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item() / args.steps
    tflops = gemm_flops(M, N, K) / ms / 1e9

    # ---- parity of what was just timed: the assembled C of the last step
    C = step()
    torch.cuda.synchronize()
    barrier()
    # (1) this rank's own column slab of its C against the CPU oracle on sampled rows of A
    rows = torch.tensor([0, 255, 256, 9999, 16384, 20000, 32767, 12345, 4097, 8191, 30000, 77, 25000, 1, 511, 31999])
    rows_d = rows.to(device)
    err, rows_checked = sampled_rows_error(C[rows_d][:, lo:hi], A[rows_d], B_shard)
    errs = torch.zeros(world, dtype=torch.float64, device=device)
    dist.all_gather_into_tensor(errs, torch.tensor([err], dtype=torch.float64, device=device))
    nan_count = torch.isnan(C[rows_d].float()).sum()
    dist.all_reduce(nan_count)
    # (2) every rank holds the same full C: position-sensitive checksums of all of C must agree
    sums = c_checksums(C)
    every = torch.zeros((world, 2), dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(every, sums.view(1, 2))
    ranks_equal = bool((every == every[0]).all().item())
    parity = {"norm_max_err": float(f"{errs.max().item():.3e}"), "tolerance": 2e-2,
              "rows_checked_per_rank": rows_checked, "columns_checked": "each rank its own slab: all N columns",
              "nan_in_sampled_rows": int(nan_count.item()), "ranks_equal": ranks_equal,
              "checksums_rank0": [int(v) for v in every[0].tolist()],
              "ok": bool(errs.max().item() <= 2e-2 and ranks_equal and int(nan_count.item()) == 0)}

    def per_rank(total_ms, steps):
        mine = torch.tensor([total_ms / steps], dtype=torch.float64, device=device)
        every_ms = torch.zeros(world, dtype=torch.float64, device=device)
        dist.all_gather_into_tensor(every_ms, mine)
        return [round(x, 4) for x in every_ms.tolist()]

    # ---- this rank's slab GEMM alone (no exchange) in alternation with cuBLAS on the same slab:
    # what the exchange costs, and whether a low per-GPU figure is this kernel or the box's state
    C_slab = torch.empty((M, hi - lo), dtype=dtype, device=device)
    C_mm = torch.empty((M, hi - lo), dtype=dtype, device=device)
    local_step = lambda: gk.gemm_tn_test(A, B_shard, C_slab)  # noqa: E731
    mm_step = lambda: torch.mm(A, B_shard.T, out=C_mm)  # noqa: E731
    local_step()
    mm_step()
    # Blocks of `steps` back-to-back launches: the fused step, this kernel alone and cuBLAS in turn,
    # twice, after a run-in of the same work that is long enough (several hundred ms) for the GPUs to
    # settle at the power cap the parity check's idle seconds lifted.  Launches timed one by one, or
    # short blocks after an idle gap, run in the boost state and make the exchange look expensive.
    for _ in range(3 * max(args.steps, 10)):
        local_step()
    # Three rounds, each starting at another variant: a block inherits the temperature its
    # predecessor left, and a fixed order would pin the hottest slot on one of the three.
    ours_ms, mm_ms, fused_ms = [], [], []
    order = [(step, fused_ms), (local_step, ours_ms), (mm_step, mm_ms)]
    for r in range(3):
        for fn, acc in order[r:] + order[:r]:
            acc.append(time_steps(fn, args.steps, torch.cuda.synchronize, barrier) / 3)
    gk.device_status()
    local_total, mm_total = sum(ours_ms), sum(mm_ms)
    t = torch.tensor([local_total, mm_total, sum(fused_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    local_ms, cublas_ms, fused_alt_ms = (t[i].item() / args.steps for i in range(3))
    local_ms_per_rank = per_rank(local_total, args.steps)
    cublas_ms_per_rank = per_rank(mm_total, args.steps)
    slab_max_diff = float((C_slab[rows_d].float() - C_mm[rows_d].float()).abs().max().item())
    del C_slab, C_mm

    # end to end: operands start in pinned host memory, the result ends there, every step.  The
    # host holds ONE copy of A, B and C between the ranks: rank g uploads its 1/G of A's rows and
    # its shard of B, the ranks replicate A over NVLink (NCCL all-gather, far faster than G
    # uploads of the whole of A over PCIe), and rank g downloads its column slab of C.
    a_lo, a_hi = rank * (M // world), (rank + 1) * (M // world)
    Ah, Bh = A[a_lo:a_hi].cpu().pin_memory(), B_shard.cpu().pin_memory()
    Ch = torch.empty((M, hi - lo), dtype=dtype).pin_memory()

    def e2e_step():
        A[a_lo:a_hi].copy_(Ah, non_blocking=True)
        B_shard.copy_(Bh, non_blocking=True)
        dist.all_gather_into_tensor(A, A[a_lo:a_hi])
        out = step()
        Ch.copy_(out[:, lo:hi], non_blocking=True)

    e2e_steps = max(2, min(args.steps, 3))
    e2e_step()
    torch.cuda.synchronize()
    e2e_total = time_steps(e2e_step, e2e_steps, torch.cuda.synchronize, barrier)
    t = torch.tensor([e2e_total], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = t.item() / e2e_steps
    gk.device_status()

    if rank == 0:
        per_gpu = tflops / world
        peak = float(peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"])
        line = {
            "metric": "bf16 GEMM TFLOP/s", "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": cfg,
            "parity": parity,
            "details": {"exchange": how, "nsplit_mode": mode, "per_gpu_tflops": round(per_gpu, 2),
                        "local_gemm_ms_per_step": round(local_ms, 4),
                        "local_gemm_note": "max over ranks of the rank's own slab GEMM without any exchange: blocks of "
                                           "`steps` back-to-back launches, in turn with blocks of the whole step and "
                                           "of cuBLAS (torch.mm) on the same slab, three blocks each with a rotating order, after a run-in",
                        "local_gemm_ms_per_rank": local_ms_per_rank,
                        "cublas_slab_ms_per_step": round(cublas_ms, 4),
                        "cublas_slab_ms_per_rank": cublas_ms_per_rank,
                        "ours_over_cublas_time": round(local_ms / cublas_ms, 4),
                        "slab_max_abs_diff_vs_cublas": slab_max_diff,
                        "step_ms_in_alternation": round(fused_alt_ms, 4),
                        "exchange_overhead": round(fused_alt_ms / local_ms - 1.0, 4),
                        "exchange_overhead_note": "step time / slowest rank's plain slab GEMM - 1, both from the blocks "
                                                  "timed in alternation after the run-in (same power state); the GPUs "
                                                  "of a box differ under the power cap and a step that ends in a "
                                                  "cross-GPU barrier runs at the slowest one's pace"},
            "e2e": {"value": round(gemm_flops(M, N, K) / e2e_ms / 1e9, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (M * K + N * K) * 2, "d2h_bytes_per_step": M * N * 2,
                    "note": "bytes summed over ranks: rank g uploads 1/G of A (replicated over NVLink by an "
                            "all-gather) and its B shard, and reads back its column slab of C",
                    "ms_per_step": round(e2e_ms, 3), "steps": e2e_steps},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clk.summary(),
            "roofline": {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": peak, "unit": "TFLOP/s",
                         "frac": round(per_gpu / peak, 4), "traffic": None,
                         "peak_source": f"{peak_src}:bf16_tflops_sustained", "kernel": "gemm_sm100::gemm_tn_fanout_kernel"
                         if mode == "fused" else "gemm_sm100::gemm_tn_kernel",
                         "note": "per-GPU TFLOP/s of the whole step (GEMM + exchange of C + barrier)"},
            "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier(device_ids=[local])
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--panels", type=int, default=8)
    ap.add_argument("--nsplit", default="auto", choices=["auto", "fused", "nccl"],
                    help="multi-GPU exchange of C: fused into the GEMM epilogue (default) or NCCL all-gather")
    ap.add_argument("--no-shapes", action="store_true", help="skip the secondary benchmark shapes")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        args.steps = args.steps or 5
        args.warmup = 1 if args.warmup is None else args.warmup
        run_reference(args, rank)
        return
    if world > 1 or args.gpus > 1:
        if world == 1:
            raise SystemExit("multi-GPU runs are launched with: python -m torch.distributed.run --nnodes=1 "
                             "--nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N")
        args.steps = args.steps or 5
        args.warmup = 3 if args.warmup is None else args.warmup
        run_multi(args)
    else:
        args.steps = args.steps or 50
        args.warmup = 5 if args.warmup is None else args.warmup
        run_single(args)


if __name__ == "__main__":
    main()
