"""Tensor-parallel execution context: how a rank combines partial results with its peers.

``NcclTpContext`` is both the baseline (plain NCCL all-reduce / all-gather after the local
GEMM, the reference's scheme: one bf16 all-reduce after o_proj, after the FFN / MoE output and
on the vocab-parallel logits, ``crates/comm/src/nccl_backend.rs``) and the home of the fused
paths. With ``fused`` on (and symmetric memory available) a row-parallel projection writes its
bf16 partial into a symmetric buffer and returns a ``PendingSum``; the RMSNorm that consumes it
runs ``parallel.fused.FusedReduce.reduce_norm``: sum over ranks through NVLink (in-switch
``multimem.ld_reduce`` or peer loads) + residual + norm + quantiser, and for larger batches the
all-gather of the quantised rows (``multimem.st``), in one kernel. Greedy selection over the
vocab-parallel lm_head exchanges one (max, index) pair per rank and row
(``FusedReduce.argmax_merge``) instead of gathering logits.

Health: every collective is followed by an async-error check when ``check_health`` is set;
a failed or timed-out collective poisons the context (all later calls raise) and the engine
latches the fault (role of ``collective_wait.rs`` and ``NcclBackend::is_healthy``).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..models.decoder import TpContext
from ..ops import Act


class CommPoisoned(RuntimeError):
    pass


class NcclTpContext(TpContext):
    def __init__(self, rank: int, size: int, device, fused: bool = True, group=None,
                 diagnostics: Optional[bool] = None):
        self.rank, self.size = rank, size
        self.device = torch.device(device)
        self.group = group
        self.fused = False
        self.poisoned: Optional[str] = None
        self.seq = 0
        self.diagnostics = (os.environ.get("METRALE_COMM_DIAGNOSTICS") == "1") if diagnostics is None else diagnostics
        self.bytes_reduced = 0
        self.reduce = None               # parallel.fused.FusedReduce once setup_fused() has run
        if os.environ.get("METRALE_NO_FUSED_COLLECTIVES") == "1":
            fused = False
        self.want_fused = bool(fused) and size > 1 and self.device.type == "cuda"

    def setup_fused(self, hidden: int, m_cap: int) -> bool:
        """Allocate the symmetric buffers of the consumer-fused reduction (collective: every rank
        calls it with the same sizes). Returns whether the fused path is on."""
        if not self.want_fused or self.reduce is not None:
            return self.reduce is not None
        try:
            from .fused import FusedReduce
            self.reduce = FusedReduce(self.rank, self.size, self.device, hidden, m_cap, self.group)
            self.fused = True
        except Exception as e:                          # symmetric memory unavailable: keep NCCL
            if self.rank == 0:
                print(f"[tp] fused reduction unavailable ({type(e).__name__}: {e}); using NCCL", flush=True)
            self.want_fused = False
        return self.reduce is not None

    def end_forward(self) -> None:
        if self.reduce is not None:
            self.reduce.end_forward()

    # ------------------------------------------------------------------ plumbing
    def _pre(self, what: str, t: torch.Tensor) -> None:
        if self.poisoned:
            raise CommPoisoned(self.poisoned)
        self.seq += 1
        if self.diagnostics:
            print(f"[comm r{self.rank}] #{self.seq} {what} {tuple(t.shape)} {t.dtype}", flush=True)

    def poison(self, reason: str) -> None:
        if not self.poisoned:
            self.poisoned = reason

    def is_healthy(self) -> bool:
        return self.poisoned is None

    def attempt_reconnect(self, timeout_s: float = 60.0) -> bool:
        """Replace a poisoned communicator: every rank must call this. A fresh process group over
        the same ranks is created (new communicator, new rendezvous keys under the same store),
        verified with one all-reduce, and swapped in; the poisoned flag is cleared only when that
        succeeds on this rank. The fused peer-memory path stays off afterwards (its symmetric
        buffers belonged to the old group). Role of ``NcclBackend::attempt_reconnect``
        (``crates/comm/src/nccl_backend.rs:254-346``: abort + re-bootstrap on master_port + 1)."""
        from datetime import timedelta
        if self.size == 1:
            self.poisoned = None
            return True
        try:
            backend = dist.get_backend(self.group) if self.group is not None else dist.get_backend()
            new_group = dist.new_group(ranks=list(range(self.size)), backend=backend,
                                       timeout=timedelta(seconds=timeout_s))
            probe = torch.ones(1, device=self.device if backend == "nccl" else "cpu")
            dist.all_reduce(probe, group=new_group)
            if int(probe.item()) != self.size:
                return False
        except RuntimeError as e:
            self.poisoned = f"reconnect failed: {e}"
            return False
        self.group, self.poisoned, self.fused, self.reconnects = new_group, None, False, getattr(self, "reconnects", 0) + 1
        self.reduce = None
        return True

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return t
        self._pre("all_reduce", t)
        try:
            dist.all_reduce(t, group=self.group)
        except RuntimeError as e:
            self.poison(f"all_reduce failed: {e}")
            raise
        self.bytes_reduced += t.numel() * t.element_size()
        return t

    def all_gather_last(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate per-rank column shards (vocab-parallel logits)."""
        if self.size == 1:
            return t
        self._pre("all_gather", t)
        parts = [torch.empty_like(t) for _ in range(self.size)]
        try:
            dist.all_gather(parts, t.contiguous(), group=self.group)
        except RuntimeError as e:
            self.poison(f"all_gather failed: {e}")
            raise
        return torch.cat(parts, dim=-1)

    def broadcast(self, t: torch.Tensor, root: int = 0) -> torch.Tensor:
        if self.size > 1:
            self._pre("broadcast", t)
            dist.broadcast(t, root, group=self.group)
        return t

    def barrier(self) -> None:
        if self.size > 1:
            dist.barrier(group=self.group)

    def linear_reduce(self, act: Act, w, residual=None, defer: bool = False):
        """Row-parallel projection: sum of the ranks' partial products, plus the residual once.
        With `defer` (and the fused reduction on) the sum is left to the norm that consumes the
        result: a ``PendingSum`` is returned instead of a tensor."""
        residual = getattr(residual, "value", residual)          # a reduced PendingSum stands for its value
        if self.size == 1:
            return ops.linear(act, w, residual=residual)
        if self.reduce is not None and act.data.is_cuda and self.reduce.supports(act.M, w.N):
            if self.poisoned:
                raise CommPoisoned(self.poisoned)
            from .fused import PendingSum
            part = self.reduce.partial_view(act.M)
            ops.linear(act, w, out=part)
            pend = PendingSum(self.reduce, part, residual)
            return pend if defer else pend.resolve()
        y = ops.linear(act, w, residual=residual if self.rank == 0 else None)
        return self.all_reduce(y)

    def sum_deferred(self, y: torch.Tensor, residual=None):
        """Sum a bf16 partial result that some other op produced (MoE experts of this rank) over
        ranks, plus the residual; deferred to the consuming norm when the fused reduction is on."""
        residual = getattr(residual, "value", residual)
        if self.size > 1 and self.reduce is not None and y.is_cuda and self.reduce.supports(y.shape[0], y.shape[1]):
            from .fused import PendingSum
            part = self.reduce.partial_view(y.shape[0])
            part.copy_(y)
            ops._count()
            return PendingSum(self.reduce, part, residual)
        y = self.all_reduce(y.to(torch.bfloat16).contiguous()) if self.size > 1 else y
        return y if residual is None else (residual.float() + y.float()).to(torch.bfloat16)


class GlooTpContext(NcclTpContext):
    """Same protocol over gloo for CPU ranks (multi-process tests of the host-side logic)."""

    def __init__(self, rank: int, size: int, group=None):
        super().__init__(rank, size, "cpu", fused=False, group=group)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return t
        self._pre("all_reduce", t)
        x = t.float() if t.dtype == torch.bfloat16 else t
        dist.all_reduce(x, group=self.group)
        if x is not t:
            t.copy_(x.to(t.dtype))
        return t

    def all_gather_last(self, t: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return t
        x = t.float().contiguous() if t.dtype == torch.bfloat16 else t.contiguous()
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x, group=self.group)
        return torch.cat(parts, dim=-1).to(t.dtype)
