"""Fused compute + collective paths over NVLink peer memory.

``FusedCollectives.gemm_allreduce`` runs a row-parallel projection whose tcgen05 GEMM kernel
also performs the all-reduce in one NVLink hop: the epilogue pushes each finished bf16 partial
tile-share into every rank's landing zone (one ``multimem.st`` through the NVSwitch multicast
mapping when the group has one, else one peer store per rank; either way overlapping the rest of
the GEMM), then
each rank sums the shares in rank order, adds the residual and stores the result into its own
rank's output buffer. Buffers live in one
symmetric allocation (``torch.distributed._symmetric_memory``: same layout on every rank, peer
pointers exchanged at rendezvous). Every device-side wait is clock-bounded and reports through
the status word. No TMA multicast and no library kernel ever touches peer memory.

The reference only ever calls ``ncclAllReduce`` after the local GEMM
(``crates/comm/src/nccl_backend/comm_impl.rs:47-94``); that path is ``NcclTpContext`` with
``fused=False`` and is the baseline these kernels are measured against.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import Act

U_CAP = 4096          # units (tile shares) per call
M_CAP = 256           # rows handled by the fused path (decode / verify batches)


class FusedCollectives:
    def __init__(self, rank: int, size: int, device, group=None, n_max: int = 8192):
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.n_max = n_max
        self.ctrl_bytes = 2 * U_CAP * 4 + 512
        self.recv_bytes = 2 * size * M_CAP * n_max * 2          # [parity][source rank][row][col]
        total = self.ctrl_bytes + self.recv_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.flags = ptrs
        self.done = [p + 2 * U_CAP * 4 for p in ptrs]
        self.par = ptrs[rank] + 2 * U_CAP * 4 + 256
        self.recv = [p + self.ctrl_bytes for p in ptrs]
        # NVLS: when the group has an NVLink multicast mapping of the allocation, the epilogue
        # broadcasts each partial with one multimem.st instead of one peer store per rank
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        mode = os.environ.get("METRALE_NVLS", "1")
        self.nvls = bool(mc) and mode != "0"
        # 2: the owner of each tile share sums all ranks' partials inside the switch
        # (multimem.ld_reduce) and broadcasts the result; 1: every rank receives every partial
        self.in_switch = self.nvls and mode == "2" and size >= 2
        self.mc_recv = (mc + self.ctrl_bytes) if self.nvls else 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)
        self.calls = 0

    def supports(self, act: Act, w) -> bool:
        return act.M <= M_CAP and w.N <= self.n_max and w.N % 128 == 0

    def gemm_allreduce(self, act: Act, w, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sum over ranks of act @ w^T (+ residual), bf16 [M, N], identical on every rank."""
        if not self.supports(act, w):
            y = ops.linear(act, w, residual=residual if self.rank == 0 else None)
            dist.all_reduce(y)
            return y
        tp = dict(size=self.size, rank=self.rank, m_cap=M_CAP, u_cap=U_CAP, recv=self.recv,
                  out=[self.mc_recv, 1 if self.in_switch else 0] + [0] * (self.size - 2), flags=self.flags, done=self.done, par=self.par)
        out = ops.linear(act, w, residual=residual, tp=tp)
        self.calls += 1
        return out
