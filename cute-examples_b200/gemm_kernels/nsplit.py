"""N-split (column-sharded B) TN GEMM over the GPUs of one node.

``C[M,N] = A[M,K] @ B[N,K].T`` with the rows of B (= columns of C) divided into one
contiguous shard per rank; A is replicated.  Rank g computes the slab
``C[:, g*N/G:(g+1)*N/G]`` with the single-GPU kernel, no operand crosses a link, and the
slabs are assembled on every rank by an all-gather of C (NCCL over NVLink on GPUs).

The reference is single-GPU and has no collective anywhere; the only thing inherited is the
per-GPU call ``gemm_tn_test(A, B_shard, C_slab)`` (kernels/gemm_kernels/__init__.cpp:6-9).

A column slab of a row-major C is not contiguous and NCCL gathers contiguous buffers, so each
rank's GEMM writes a contiguous staging slab ``[rows, N/G]``, the all-gather fills
``[G, rows, N/G]``, and one strided copy lays it out as ``C[rows, N]``.  The rows of C are
processed in panels so that panel p's all-gather and copy (communication stream) run under
panel p+1's GEMM (compute stream).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def shard_rows(n: int, world_size: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the rows of B (columns of C) that `rank` owns.  Shards are equal
    (all-gather needs equal counts) and a multiple of 8 columns (16-byte row pitch)."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if n % world_size != 0:
        raise ValueError(f"N={n} must be divisible by the number of ranks ({world_size})")
    per = n // world_size
    if per % 8 != 0:
        raise ValueError(f"N/ranks={per} must be a multiple of 8")
    return rank * per, (rank + 1) * per


@dataclass
class NSplitPlan:
    """Row panels of C and the buffers one rank needs; built once, reused every call."""
    M: int
    N: int
    world_size: int
    panel_rows: int
    staging: list            # 2 x [panel_rows, N/G]      local slab of one panel
    gathered: list           # 2 x [G, panel_rows, N/G]   all ranks' slabs of one panel

    @property
    def shard_cols(self) -> int:
        return self.N // self.world_size

    @property
    def num_panels(self) -> int:
        return (self.M + self.panel_rows - 1) // self.panel_rows

    @staticmethod
    def create(M: int, N: int, world_size: int, dtype: torch.dtype, device, num_panels: int = 8,
               row_multiple: int = 256) -> "NSplitPlan":
        shard_rows(N, world_size, 0)
        num_panels = max(1, min(num_panels, max(1, M // row_multiple)))
        rows = (M + num_panels - 1) // num_panels
        rows = ((rows + row_multiple - 1) // row_multiple) * row_multiple if M >= row_multiple else M
        per = N // world_size
        staging = [torch.empty((rows, per), dtype=dtype, device=device) for _ in range(2)]
        gathered = [torch.empty((world_size, rows, per), dtype=dtype, device=device) for _ in range(2)]
        return NSplitPlan(M, N, world_size, rows, staging, gathered)


def gemm_tn_nsplit(A: torch.Tensor, B_shard: torch.Tensor, C: torch.Tensor,
                   group: Optional[dist.ProcessGroup] = None, plan: Optional[NSplitPlan] = None,
                   local_gemm: Optional[Callable] = None, comm_stream=None) -> torch.Tensor:
    """Computes the full ``C[M,N]`` on every rank of `group`.

    A: [M,K] (same on every rank); B_shard: this rank's rows of B, [N/G,K]; C: [M,N] output.
    `local_gemm(A_rows, B_shard, C_slab)` defaults to the sm_100a kernel; tests that run on CPU
    ranks pass an fp32 matmul instead.  Every rank validates its arguments BEFORE the first
    collective, so a bad rank raises instead of leaving its peers inside an all-gather.
    """
    world = dist.get_world_size(group)
    M, K = A.shape
    per, Kb = B_shard.shape
    N = per * world
    if Kb != K:
        raise ValueError(f"inner dimensions differ: A has K={K}, B shard has K={Kb}")
    if tuple(C.shape) != (M, N):
        raise ValueError(f"C must be [{M}, {N}], got {tuple(C.shape)}")
    if not C.is_contiguous():
        raise ValueError("C must be contiguous")
    if plan is None:
        plan = NSplitPlan.create(M, N, world, C.dtype, C.device)
    if (plan.M, plan.N, plan.world_size) != (M, N, world):
        raise ValueError("plan was built for another problem")
    if local_gemm is None:
        from . import gemm_tn_test as local_gemm  # the product path; no fallback

    on_gpu = C.is_cuda
    if on_gpu:
        compute = torch.cuda.current_stream(C.device)
        comm = comm_stream if comm_stream is not None else _comm_stream(C.device)
        comm.wait_stream(compute)
    done_events = [None, None]   # staging/gathered buffer i is free again after this event

    for p in range(plan.num_panels):
        r0 = p * plan.panel_rows
        r1 = min(M, r0 + plan.panel_rows)
        rows = r1 - r0
        slot = p & 1
        stage = plan.staging[slot][:rows]
        gath = plan.gathered[slot].view(-1)[: world * rows * per].view(world, rows, per)
        if on_gpu and done_events[slot] is not None:
            compute.wait_event(done_events[slot])
        local_gemm(A[r0:r1], B_shard, stage)
        if on_gpu:
            ready = torch.cuda.Event()
            ready.record(compute)
            comm.wait_event(ready)
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(gath.view(world * rows, per), stage, group=group)
                C[r0:r1].view(rows, world, per).copy_(gath.permute(1, 0, 2))
                ev = torch.cuda.Event()
                ev.record(comm)
            done_events[slot] = ev
        else:
            dist.all_gather_into_tensor(gath.view(world * rows, per), stage.contiguous(), group=group)
            C[r0:r1].view(rows, world, per).copy_(gath.permute(1, 0, 2))
    if on_gpu:
        compute.wait_stream(comm)
    return C


def fanout_pointers(buffer_ptrs, rank: int, column_offset: int, element_size: int) -> list:
    """Device addresses rank `rank` stores its column slab to: the same column offset inside every
    GPU's C.  Its own copy comes first (the local store does not wait behind the link), then the
    peers in ring order rank+1, rank+2, ...: at any moment the ranks then aim at different
    destination GPUs instead of all writing to GPU 0, then GPU 1, and so on."""
    world = len(buffer_ptrs)
    if not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for {world} buffers")
    order = [(rank + i) % world for i in range(world)]
    return [int(buffer_ptrs[r]) + column_offset * element_size for r in order]


class FusedNSplit:
    """Column-sharded GEMM with the all-gather of C folded into the GEMM epilogue.

    Every rank owns full ``C[M, N]`` buffers in symmetric memory (same allocation on every GPU,
    mapped into every process).  Rank g computes its column slab ``A @ B_g.T`` once and its epilogue
    stores every finished tile into all G copies of C (one TMA store per GPU per tile: the local
    one and G-1 over NVLink), at column offset ``g * N/G``.  No staging slab, no NCCL all-gather,
    no re-stride copy.  Peer memory is only ever written, never loaded from.

    Synchronisation: ONE cross-GPU barrier per call, after the GEMM (everybody's stores have
    landed).  The barrier that would have to precede the GEMM (nobody still reads the C that is
    about to be overwritten) is made unnecessary by alternating between ``buffers`` = 2 copies of
    C: call t writes copy t % 2; a peer can start writing into this rank's copy t % 2 only after it
    has passed the barrier of call t-1, which this rank enters, in stream order, after its own
    call t-1 and therefore after everything it enqueued to read the result of call t-2.
    So: the tensor a call returns stays valid until the call after the next one, and must be
    read by work enqueued (on the calling stream) before this rank's next call.  With
    ``buffers=1`` there is one copy of C and two barriers per call.
    """

    def __init__(self, M: int, N: int, dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None,
                 buffers: int = 2):
        import torch.distributed._symmetric_memory as symm_mem

        if buffers not in (1, 2):
            raise ValueError("buffers must be 1 or 2")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.M, self.N = M, N
        self.lo, self.hi = shard_rows(N, self.world, self.rank)
        if self.world > 8:
            raise ValueError("the fused exchange stores to at most 8 GPUs")
        self.storage = symm_mem.empty((buffers, M, N), dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.storage, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned an unexpected number of buffers")
        esize = self.storage.element_size()
        self.copies = [self.storage[i] for i in range(buffers)]
        self.output_ptrs = [fanout_pointers([p + i * M * N * esize for p in ptrs], self.rank, self.lo, esize)
                            for i in range(buffers)]
        self.calls = 0
        self.C = self.copies[0]

    def __call__(self, A: torch.Tensor, B_shard: torch.Tensor) -> torch.Tensor:
        from . import gemm_tn_fanout

        if tuple(A.shape) != (self.M, B_shard.shape[1]) or B_shard.shape[0] != self.hi - self.lo:
            raise ValueError(f"expected A [{self.M}, K] and B shard [{self.hi - self.lo}, K], got "
                             f"{tuple(A.shape)} and {tuple(B_shard.shape)}")
        which = self.calls % len(self.copies)
        self.calls += 1
        if len(self.copies) == 1:
            self.handle.barrier(channel=0)
        gemm_tn_fanout(A, B_shard, self.output_ptrs[which], self.N)
        self.handle.barrier(channel=1)
        self.C = self.copies[which]
        return self.C


_COMM_STREAMS: dict = {}


def _comm_stream(device):
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device=key)
    return _COMM_STREAMS[key]
