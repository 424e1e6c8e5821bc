"""Timing table of the column-sharded (N-split) GEMM on the GPUs of one node.

Launched with one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port P \\
        cute-examples_b200/tests/nsplit_bench.py [--n 32768] [--variants fused,fused_c0,fused_c1,fused_1buf,nccl8,local,mm]

Variants (timed in alternation, every round starting at another variant, `--rounds` rounds of `--iters`
steps, CUDA events, max over ranks):
    fused       FusedNSplit as the library configures it (two copies of C, one barrier per step)
    fused_c0    the same with the 256 x 256 pair tile forced;  fused_c1: the 256 x 512 tile forced
    fused_1buf  one copy of C, a barrier before and after the GEMM
    nccl8       per-panel GEMM + NCCL all-gather + re-stride copy, 8 row panels
    local       this rank's slab GEMM alone, no exchange;  mm: cuBLAS (torch.mm) on the same slab
The reference is single-GPU and has no counterpart (kernels/tests/gemm_bench.py times one GPU).

`--emulate-outputs 8` (any G >= 2): every rank runs the slab GEMM of an 8-GPU split (N / 8 columns) and its
epilogue stores every tile once locally and 7 times into peer memory (slabs 1..7 of the next
rank's buffer), i.e. the NVLink store load of one GPU of an 8-GPU run, on two GPUs.  The slabs are
compared with the plain kernel's result afterwards.
"""
import argparse
import json
import os
import statistics
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import gemm_kernels as gk  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=32768)
    ap.add_argument("--n", type=int, default=32768)
    ap.add_argument("--k", type=int, default=32768)
    ap.add_argument("--variants", default="fused,fused_c0,fused_c1,fused_1buf,nccl8,local,mm")
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--emulate-outputs", type=int, default=0)
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    M, N, K = args.m, args.n, args.k
    dtype = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(4)
    A = torch.empty((M, K), dtype=dtype, device=device)
    for r0 in range(0, M, 4096):
        A[r0:r0 + 4096] = (torch.randn((min(4096, M - r0), K), generator=g, device=device) / K ** 0.5).to(dtype)

    def timed(fn, iters):
        torch.cuda.synchronize()
        dist.barrier(device_ids=[local])
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], dtype=torch.float64, device=device)
        every = torch.zeros(world, dtype=torch.float64, device=device)
        dist.all_gather_into_tensor(every, t)
        return every.tolist()

    calls = {}
    if args.emulate_outputs:
        import torch.distributed._symmetric_memory as symm_mem

        outs = args.emulate_outputs
        per = N // outs
        gb = torch.Generator(device=device).manual_seed(4000 + rank)
        B_shard = (torch.randn((per, K), generator=gb, device=device) / K ** 0.5).to(dtype)
        buf = symm_mem.empty((M, outs * per), dtype=dtype, device=device)
        handle = symm_mem.rendezvous(buf, dist.group.WORLD)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        peer = (rank + 1) % world
        targets = [ptrs[rank]] + [ptrs[peer] + j * per * 2 for j in range(1, outs)]
        local_only = [ptrs[rank] + j * per * 2 for j in range(outs)]
        C_plain = torch.empty((M, per), dtype=dtype, device=device)

        def fan(where):
            def f():
                gk.gemm_tn_fanout(A, B_shard, where, outs * per)
                handle.barrier(channel=1)
            return f

        # variant -> (forced tile configuration or -1, step)
        calls = {"peer_auto": (-1, fan(targets)), "peer_c0": (0, fan(targets)), "peer_c1": (1, fan(targets)),
                 "local_c0": (0, fan(local_only)), "local_c1": (1, fan(local_only)),
                 "plain": (-1, lambda: gk.gemm_tn_test(A, B_shard, C_plain)),
                 "mm": (-1, lambda: torch.mm(A, B_shard.T, out=C_plain))}
    else:
        lo, hi = gk.shard_rows(N, world, rank)
        gb = torch.Generator(device=device).manual_seed(4000 + rank)
        B_shard = (torch.randn((hi - lo, K), generator=gb, device=device) / K ** 0.5).to(dtype)
        wanted = [v.strip() for v in args.variants.split(",") if v.strip()]
        C_slab = torch.empty((M, hi - lo), dtype=dtype, device=device)
        if any(v.startswith("fused") and v != "fused_1buf" for v in wanted):
            fused2 = gk.FusedNSplit(M, N, dtype, device, buffers=2)
        if "fused_1buf" in wanted:
            fused1 = gk.FusedNSplit(M, N, dtype, device, buffers=1)
        if "nccl8" in wanted:
            C_full = torch.empty((M, N), dtype=dtype, device=device)
            plan8 = gk.NSplitPlan.create(M, N, world, dtype, device, num_panels=8)

        for v in wanted:
            if v == "fused":
                calls[v] = (-1, lambda: fused2(A, B_shard))
            elif v == "fused_c0":
                calls[v] = (0, lambda: fused2(A, B_shard))
            elif v == "fused_c1":
                calls[v] = (1, lambda: fused2(A, B_shard))
            elif v == "fused_1buf":
                calls[v] = (-1, lambda: fused1(A, B_shard))
            elif v == "nccl8":
                calls[v] = (-1, lambda: gk.gemm_tn_nsplit(A, B_shard, C_full, plan=plan8))
            elif v == "local":
                calls[v] = (-1, lambda: gk.gemm_tn_test(A, B_shard, C_slab))
            elif v == "mm":
                calls[v] = (-1, lambda: torch.mm(A, B_shard.T, out=C_slab))
            else:
                raise SystemExit(f"unknown variant {v}")

    res = {k: [] for k in calls}
    for k, (cfg, fn) in calls.items():
        gk.set_option("tile_config", cfg)
        fn()
    order = list(calls.items())
    for r in range(args.rounds):
        # every round starts at another variant: in the power-capped state a variant inherits the
        # temperature its predecessor left, and a fixed order would pin that on one of them
        for k, (cfg, fn) in order[r % len(order):] + order[:r % len(order)]:
            gk.set_option("tile_config", cfg)          # once per measurement, not per step
            res[k].append(timed(fn, args.iters))
    gk.set_option("tile_config", -1)
    gk.device_status()

    check = None
    if args.emulate_outputs:
        gk.gemm_tn_test(A, B_shard, C_plain)
        calls["peer_auto"][1]()
        torch.cuda.synchronize()
        dist.barrier(device_ids=[local])
        # slab 0 of my buffer is my own product; slabs 1.. hold the previous rank's product
        mine = torch.equal(buf[:, :per].contiguous().view(torch.int16), C_plain.view(torch.int16))
        sums = torch.stack([buf[:, j * per:(j + 1) * per].contiguous().view(torch.int16).to(torch.int64).sum()
                            for j in range(outs)])
        plain_sum = C_plain.view(torch.int16).to(torch.int64).sum().view(1)
        every = torch.zeros(world, dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(every, plain_sum)
        prev = (rank - 1) % world
        check = bool(mine and bool((sums[1:] == every[prev]).all().item()))
        flags = torch.zeros(world, dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(flags, torch.tensor([int(check)], dtype=torch.int64, device=device))
        check = bool(flags.min().item() == 1)

    if rank == 0:
        flops = 2.0 * M * (N // args.emulate_outputs if args.emulate_outputs else N) * K
        table = {}
        for k, rounds in res.items():
            worst = [max(r) for r in rounds]                      # max over ranks per round
            table[k] = {"ms": round(statistics.median(worst), 3), "min_ms": round(min(worst), 3),
                        "per_rank_ms": [round(statistics.median(r[i] for r in rounds), 3) for i in range(world)]}
            if not args.emulate_outputs and k not in ("local", "mm"):
                table[k]["aggregate_tflops"] = round(flops / statistics.median(worst) / 1e9, 1)
        print(json.dumps({"world": world, "M": M, "N": N, "K": K, "emulate_outputs": args.emulate_outputs,
                          "rounds": args.rounds, "iters": args.iters, "slabs_match_plain_kernel": check,
                          "variants": table}), flush=True)
        for k, v in table.items():
            print(f"{k:>11}: {v['ms']:9.3f} ms (min {v['min_ms']:.3f})  per rank {v['per_rank_ms']}", flush=True)
    dist.barrier(device_ids=[local])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
