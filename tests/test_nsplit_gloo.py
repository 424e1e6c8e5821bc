"""N-split sharding / assembly logic on CPU ranks (gloo, world size 2): the per-GPU GEMM is
replaced by an fp32 CPU matmul of the shard, everything else is the product's code path."""
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_ROOT, REPO


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_gemm(A, B, C):
    C.copy_(torch.matmul(A.float(), B.float().T).to(C.dtype))
    return C


def _worker(rank, world, port, scenario, q):
    try:
        for p in (str(REPO), str(PKG_ROOT)):
            if p not in sys.path:
                sys.path.insert(0, p)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import datetime

        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
        from gemm_kernels import NSplitPlan, gemm_tn_nsplit, shard_rows
        from oracle import oracle

        if scenario == "assemble":
            M, N, K = 96, 64, 40
            A, B = oracle.make_inputs(M, N, K, 70)
            lo, hi = shard_rows(N, world, rank)
            C = torch.full((M, N), float("nan"), dtype=torch.bfloat16)
            plan = NSplitPlan.create(M, N, world, torch.bfloat16, "cpu", num_panels=3, row_multiple=16)
            assert plan.num_panels == 3
            gemm_tn_nsplit(A, B[lo:hi].contiguous(), C, plan=plan, local_gemm=_cpu_gemm)
            want = torch.matmul(A.float(), B.float().T).to(torch.bfloat16)
            ok = torch.equal(C.view(torch.int16), want.view(torch.int16))
            # ragged last panel
            M2 = 100
            A2, _ = oracle.make_inputs(M2, N, K, 71)
            C2 = torch.full((M2, N), float("nan"), dtype=torch.bfloat16)
            plan2 = NSplitPlan.create(M2, N, world, torch.bfloat16, "cpu", num_panels=3, row_multiple=16)
            gemm_tn_nsplit(A2, B[lo:hi].contiguous(), C2, plan=plan2, local_gemm=_cpu_gemm)
            want2 = torch.matmul(A2.float(), B.float().T).to(torch.bfloat16)
            ok = ok and torch.equal(C2.view(torch.int16), want2.view(torch.int16))
            q.put((rank, "ok" if ok else "mismatch"))
        elif scenario == "bad_rank_raises_before_collective":
            # rank 1 passes a C of the wrong shape: it must raise on its own, before any
            # collective, and rank 0 must not be left waiting inside an all-gather.
            M, N, K = 32, 32, 16
            A, B = oracle.make_inputs(M, N, K, 72)
            lo, hi = shard_rows(N, world, rank)
            C = torch.empty((M, N if rank == 0 else N + 8), dtype=torch.bfloat16)
            try:
                if rank == 1:
                    gemm_tn_nsplit(A, B[lo:hi].contiguous(), C, local_gemm=_cpu_gemm)
                    q.put((rank, "no error"))
                else:
                    q.put((rank, "ok"))          # rank 0 does not enter the collective in this scenario
            except ValueError as e:
                q.put((rank, "ok" if "C must be" in str(e) else f"wrong error {e}"))
        dist.destroy_process_group()
    except Exception:  # pragma: no cover
        q.put((rank, traceback.format_exc()))


@pytest.mark.parametrize("scenario", ["assemble", "bad_rank_raises_before_collective"])
def test_nsplit_two_cpu_ranks(scenario):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def test_shard_rows():
    from gemm_kernels import shard_rows

    assert shard_rows(32768, 8, 3) == (12288, 16384)
    assert [shard_rows(64, 2, r) for r in range(2)] == [(0, 32), (32, 64)]
    with pytest.raises(ValueError):
        shard_rows(100, 8, 0)
    with pytest.raises(ValueError):
        shard_rows(48, 4, 0)       # 12 columns per rank: not a multiple of 8
    with pytest.raises(ValueError):
        shard_rows(64, 2, 2)


def test_fanout_pointers():
    from gemm_kernels import fanout_pointers, shard_rows

    bufs = [0x1000_0000, 0x2000_0000, 0x3000_0000, 0x4000_0000]
    lo, _ = shard_rows(32768, 4, 2)
    ptrs = fanout_pointers(bufs, 2, lo, 2)
    assert ptrs[0] == 0x3000_0000 + lo * 2                       # own copy first
    assert sorted(p - lo * 2 for p in ptrs) == bufs              # every GPU exactly once
    assert all(p % 16 == 0 for p in ptrs)                        # slab starts stay 16-byte aligned
    with pytest.raises(ValueError):
        fanout_pointers(bufs, 4, 0, 2)
