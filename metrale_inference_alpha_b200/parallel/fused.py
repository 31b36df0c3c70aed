"""Fused compute + collective paths over NVLink peer memory.

``FusedReduce`` holds the symmetric buffers and barrier state of one tensor-parallel group
(``torch.distributed._symmetric_memory``: same layout on every rank, peer pointers and the
NVLink multicast alias exchanged at rendezvous) for the kernels in ``ops/csrc/tp_fused.cu``: a
row-parallel projection writes its bf16 partial into a symmetric buffer, and the RMSNorm +
quantiser that consumes it performs the sum over ranks itself (in-switch ``multimem.ld_reduce``,
or peer loads), adds the residual, normalises, quantises and, for larger batches, broadcasts the
quantised rows with ``multimem.st`` so that the next GEMM reads the gathered operand from local
memory. Every device-side wait is clock-bounded and reports through the status word. No TMA
multicast and no library kernel ever touches peer memory.

The reference only ever calls ``ncclAllReduce`` after the local GEMM and runs the norm as its
own kernel (``crates/comm/src/nccl_backend/comm_impl.rs:47-94``); that path is
``NcclTpContext`` with ``fused=False`` and is the baseline these kernels are measured against.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import Act


# ======================================================================================
# Consumer-fused reduction: all-reduce + residual + RMSNorm + quantiser (+ all-gather)
# ======================================================================================
import ctypes as C  # noqa: E402

from ..ops import _native  # noqa: E402

_VP8 = C.c_void_p * 8


class TpSyncArgs(C.Structure):
    _fields_ = [("arrive", C.c_void_p), ("arrive_mc", C.c_void_p), ("arrive_peer", _VP8),
                ("done", C.c_void_p), ("done_mc", C.c_void_p), ("done_peer", _VP8),
                ("epoch", C.c_void_p), ("cta_done", C.c_void_p), ("status", C.c_void_p),
                ("wait_cycles", C.c_longlong), ("size", C.c_int), ("rank", C.c_int)]


class TpNormArgs(C.Structure):
    _fields_ = [("sync", TpSyncArgs), ("M", C.c_int), ("K", C.c_int), ("two_shot", C.c_int), ("out_mode", C.c_int),
                ("partial_mc", C.c_void_p), ("partial", _VP8), ("residual", C.c_void_p),
                ("residual_out", C.c_void_p), ("residual_out_mc", C.c_void_p), ("w", C.c_void_p),
                ("do_norm", C.c_int), ("w_plus_one", C.c_int), ("eps", C.c_float),
                ("out", C.c_void_p), ("out_ld", C.c_longlong), ("out_bf16", C.c_void_p), ("out_bf16_ld", C.c_longlong),
                ("scale", C.c_void_p), ("scale_ld", C.c_int), ("sf", C.c_void_p), ("sf_k64", C.c_int),
                ("static_gs", C.c_float), ("max_ctas", C.c_int),
                ("ll", C.c_void_p), ("ll_mc", C.c_void_p), ("ll_peer", _VP8), ("ll_rows", C.c_int)]


class TpMergeArgs(C.Structure):
    _fields_ = [("sync", TpSyncArgs), ("M", C.c_int), ("pairs", _VP8), ("out_ids", C.c_void_p), ("feed", C.c_void_p)]


_native.register_optional("mb_tp_reduce_norm", [C.POINTER(TpNormArgs), C.c_void_p])
_native.register_optional("mb_tp_argmax_merge", [C.POINTER(TpMergeArgs), C.c_void_p])
_native.register_optional("mb_tp_barrier", [C.POINTER(TpSyncArgs), C.c_void_p])
_native.register_optional("mb_argmax_shard", [C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int, C.c_void_p,
                                              C.c_int, C.c_void_p])

OUT_NONE = 4


class PendingSum:
    """The output of a row-parallel projection before it has been summed over ranks: this rank's
    bf16 partial (in the symmetric partial buffer) and the residual it will be added to. The
    RMSNorm that consumes it performs the sum (``FusedReduce.reduce_norm``); ``value`` is the
    summed residual stream afterwards. With ``rows_valid`` < M only this rank's row share of
    ``value`` is meaningful (two-shot protocol without a residual gather), which is all the next
    reduction needs."""

    def __init__(self, owner: "FusedReduce", partial: torch.Tensor, residual: Optional[torch.Tensor]):
        self.owner, self.partial, self.residual = owner, partial, residual
        self.value: Optional[torch.Tensor] = None
        self.full = False
        self.shape, self.dtype, self.device, self.is_cuda = partial.shape, partial.dtype, partial.device, True

    def resolve(self) -> torch.Tensor:
        """The summed tensor on every rank (no norm)."""
        if self.value is None or not self.full:
            if self.value is not None:
                raise RuntimeError("a row-share-only reduction cannot be widened afterwards")
            self.owner.reduce_norm(self, None, "none", gather_residual=True, do_norm=False)
        return self.value


class FusedReduce:
    """Symmetric buffers + barrier state of one tensor-parallel group for the consumer-fused
    reduction (``ops/csrc/tp_fused.cu``). Works with world size 1 (loop-back) for single-GPU
    tests; ``emulate`` > 1 sums that many local partial buffers on one GPU through the peer-load
    path (the barrier then counts this rank's own signals)."""

    def __init__(self, rank: int, size: int, device, hidden: int, m_cap: int, group=None,
                 emulate: int = 0, use_multicast: Optional[bool] = None, wait_cycles: int = 0):
        self.rank, self.size, self.device = rank, size, torch.device(device)
        self.hidden, self.m_cap = hidden, m_cap
        self.emulate = emulate
        self.wait_cycles = wait_cycles
        K = hidden
        self.sf_k64 = ((K + 255) // 256) * 4
        n_ranks = max(size, emulate, 1)
        al = lambda n: (n + 255) // 256 * 256
        self.scale_ld = (m_cap + 63) // 64 * 64
        self.ll_rows = min(m_cap, 64)
        lay, o = {}, 0
        for name, n in (("sync", 1024), ("pairs", 2 * m_cap * 8),
                        ("ll", 2 * max(size, 1) * self.ll_rows * (K // 2) * 8),
                        ("partial", 2 * m_cap * K * 2 * (emulate if emulate > 1 else 1)),
                        ("data", m_cap * K * 2), ("bf16", m_cap * K * 2), ("resid", m_cap * K * 2),
                        ("sf", ((m_cap + 127) // 128) * self.sf_k64 * 512),
                        ("scale", max(m_cap, ((K + 127) // 128) * self.scale_ld) * 4)):
            lay[name] = (o, n)
            o += al(n)
        self.lay, total = lay, o
        self.mc = 0
        if size > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            if use_multicast is None:
                use_multicast = os.environ.get("METRALE_NVLS", "1") != "0"
            self.mc = mc if use_multicast else 0
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()] * n_ranks
        self._view("scale", torch.float32).fill_(1.0)
        self.local = torch.zeros(8, dtype=torch.int32, device=self.device)      # epoch[2], cta_done
        self.calls = 0
        self.pair_calls = 0
        self.dirty = False               # a one-shot reduction has run since the last full barrier
        # one-shot while the partials every GPU must serve to all readers stay small (size x M x K x 2
        # bytes leave each GPU per call); above that the row-owner protocol moves 1 / size of it
        # (measured crossovers: ~3.7 MB on 8 GPUs, above 6 MB on 2)
        self.one_shot_bytes = int(os.environ.get("METRALE_TP_ONESHOT_BYTES", str((8 << 20) if size <= 2 else (3584 << 10))))
        # packet protocol (no barrier, one NVLink hop, twice the bytes): measured faster than the
        # barrier one-shot only between two ranks and below ~400 KB received per call
        self.packet_bytes = int(os.environ.get("METRALE_TP_PACKET_BYTES", str((400 << 10) if size <= 2 else 0)))
        self.force_proto: Optional[int] = None            # tests: 0 one-shot, 1 two-shot, 2 packets
        torch.cuda.synchronize(self.device)
        if size > 1:
            dist.barrier(group=group)

    # ------------------------------------------------------------------ layout
    def _view(self, name: str, dtype, parity: int = 0, nbuf: int = 1) -> torch.Tensor:
        o, n = self.lay[name]
        n //= nbuf
        return self.buf[o + parity * n: o + (parity + 1) * n].view(dtype)

    def _addr(self, base: int, name: str, parity: int = 0, nbuf: int = 1) -> int:
        o, n = self.lay[name]
        return base + o + parity * (n // nbuf)

    def _sync(self, status_ptr) -> TpSyncArgs:
        s = TpSyncArgs()
        n = max(self.size, self.emulate, 1)
        me = self.ptrs[self.rank if self.size > 1 else 0]
        s.arrive, s.done = me + self.lay["sync"][0], me + self.lay["sync"][0] + 256
        if self.mc:
            s.arrive_mc, s.done_mc = self.mc + self.lay["sync"][0], self.mc + self.lay["sync"][0] + 256
        for r in range(n):
            s.arrive_peer[r] = self.ptrs[r] + self.lay["sync"][0]
            s.done_peer[r] = self.ptrs[r] + self.lay["sync"][0] + 256
        s.epoch, s.cta_done = self.local.data_ptr(), self.local.data_ptr() + 16
        s.status = status_ptr
        s.wait_cycles = self.wait_cycles
        s.size, s.rank = n, self.rank
        return s

    # ------------------------------------------------------------------ producer side
    def supports(self, M: int, N: int) -> bool:
        return M <= self.m_cap and N == self.hidden and N % 64 == 0 and N <= 8192

    def partial_view(self, M: int, slot: int = 0) -> torch.Tensor:
        """Where the next row-parallel GEMM writes this rank's partial [M, hidden] bf16. `slot`
        selects one of `emulate` local buffers in single-GPU emulation."""
        par = self.calls & 1
        nb = 2 * (self.emulate if self.emulate > 1 else 1)
        v = self._view("partial", torch.bfloat16, par * (nb // 2) + slot, nb)
        return v[:M * self.hidden].view(M, self.hidden)

    def protocol(self, M: int, K: int) -> int:
        """0 one-shot behind a barrier, 1 two-shot (row owners + multicast gather), 2 packets."""
        if self.force_proto is not None:
            return self.force_proto
        n = max(self.size, 1)
        if self.emulate <= 1 and M <= self.ll_rows and n * M * K * 4 <= self.packet_bytes:
            return 2
        if self.size > 1 and self.mc and self.size * M * K * 2 > self.one_shot_bytes:
            return 1
        return 0

    # ------------------------------------------------------------------ consumer side
    def reduce_norm(self, pend: PendingSum, w: Optional[torch.Tensor], fmt: str, *, plus_one: bool = False,
                    eps: float = 1e-6, also_bf16: bool = False, gather_residual: bool = False,
                    do_norm: bool = True, static_scale: float = 0.0) -> Optional[Act]:
        """Sum `pend` over ranks, add its residual, (RMS-)normalise and encode as `fmt`
        ("bf16" | "fp8_row" | "fp8_g128" | "nvfp4" | "none"). Sets pend.value."""
        M, K = pend.partial.shape
        rt = ops.runtime(self.device)
        n = max(self.size, self.emulate, 1)
        proto = self.protocol(M, K)
        two = proto == 1
        a = TpNormArgs()
        a.sync = self._sync(rt.status.data_ptr())
        a.M, a.K, a.two_shot = M, K, proto
        if proto == 2:
            me = self.ptrs[self.rank if self.size > 1 else 0]
            a.ll, a.ll_rows = self._addr(me, "ll"), self.ll_rows
            if self.mc:
                a.ll_mc = self._addr(self.mc, "ll")
            for r in range(max(self.size, 1)):
                a.ll_peer[r] = self._addr(self.ptrs[r], "ll")
        par = self.calls & 1
        nb = 2 * (self.emulate if self.emulate > 1 else 1)
        if self.mc:
            a.partial_mc = self._addr(self.mc, "partial", par, 2)
        for r in range(n):
            if self.emulate > 1:
                a.partial[r] = self._addr(self.ptrs[0], "partial", par * (nb // 2) + r, nb)
            else:
                a.partial[r] = self._addr(self.ptrs[r], "partial", par, 2)
        out_base = self.mc if two else self.ptrs[self.rank if self.size > 1 else 0]
        if pend.residual is not None:
            a.residual = pend.residual.data_ptr()
        if two and gather_residual:
            value = self._view("resid", torch.bfloat16)[:M * K].view(M, K)
            a.residual_out_mc = self._addr(self.mc, "resid")
            full = True
        else:
            value = torch.empty(M, K, dtype=torch.bfloat16, device=self.device)
            a.residual_out = value.data_ptr()
            full = not two
        a.w = w.data_ptr() if w is not None else None
        a.do_norm, a.w_plus_one, a.eps = int(do_norm), int(plus_one), eps
        act = None
        if fmt == "none":
            a.out_mode = OUT_NONE
        else:
            a.out_mode = ops.OUT_MODE[fmt]
            act = Act(fmt, M, K, None)
            if fmt == "bf16":
                act.data = self._view("data", torch.bfloat16)[:M * K].view(M, K)
                act.bf16 = act.data
                a.out_ld = K
            elif fmt == "fp8_row":
                act.data = self._view("data", torch.uint8)[:M * K].view(M, K)
                act.scale = self._view("scale", torch.float32)[:M]
                a.out_ld = K
            elif fmt == "fp8_g128":
                act.data = self._view("data", torch.uint8)[:M * K].view(M, K)
                act.scale = self._view("scale", torch.float32)[:((K + 127) // 128) * self.scale_ld].view(-1, self.scale_ld)
                a.out_ld, a.scale_ld = K, self.scale_ld
            else:
                act.data = self._view("data", torch.uint8)[:M * (K // 2)].view(M, K // 2)
                act.scale = self._view("scale", torch.float32)[:M]
                act.sf = self._view("sf", torch.uint8)
                act.sf_k64 = self.sf_k64
                a.out_ld, a.sf_k64 = K // 2, self.sf_k64
                a.sf = self._addr(out_base, "sf")
                a.static_gs = float(static_scale)
            a.out = self._addr(out_base, "data")
            a.scale = self._addr(out_base, "scale")
            if also_bf16 and fmt != "bf16":
                act.bf16 = self._view("bf16", torch.bfloat16)[:M * K].view(M, K)
                a.out_bf16, a.out_bf16_ld = self._addr(out_base, "bf16"), K
        _native.check(_native.lib().mb_tp_reduce_norm(C.byref(a), ops._stream()), "tp_reduce_norm")
        ops._count()
        self.calls += 1
        self.dirty = proto == 0                 # only the barrier one-shot leaves peers reading this rank's partial
        pend.value, pend.full = value, full
        return act

    def argmax_merge(self, logits: torch.Tensor, vocab_lo: int, out: torch.Tensor,
                     feed: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Greedy token ids from vocabulary-sharded logits [M, V / size]: per-rank argmax, then a
        merge of one (max, global index) pair per rank and row pulled over NVLink."""
        M, V = logits.shape
        assert M <= self.m_cap
        rt = ops.runtime(self.device)
        par = self.pair_calls & 1
        L = _native.lib()
        mine = self.ptrs[self.rank if self.size > 1 else 0]
        _native.check(L.mb_argmax_shard(logits.data_ptr(), int(logits.dtype == torch.float32), logits.stride(0), M, V,
                                        self._addr(mine, "pairs", par, 2), int(vocab_lo), ops._stream()), "argmax_shard")
        a = TpMergeArgs()
        a.sync = self._sync(rt.status.data_ptr())
        a.M = M
        for r in range(max(self.size, 1)):
            a.pairs[r] = self._addr(self.ptrs[r], "pairs", par, 2)
        a.out_ids = out.data_ptr()
        a.feed = feed.data_ptr() if feed is not None else None
        _native.check(L.mb_tp_argmax_merge(C.byref(a), ops._stream()), "tp_argmax_merge")
        ops._count(2)
        self.pair_calls += 1
        self.dirty = False
        return out

    def barrier(self) -> None:
        s = self._sync(ops.runtime(self.device).status.data_ptr())
        _native.check(_native.lib().mb_tp_barrier(C.byref(s), ops._stream()), "tp_barrier")
        ops._count()
        self.dirty = False

    def end_forward(self) -> None:
        """Close a forward pass: when its last reduction was one-shot (no exit barrier), a barrier
        orders every rank's reads of the partial buffers before the next pass overwrites them."""
        if self.dirty and self.size > 1:
            self.barrier()
        self.dirty = False
        if self.calls & 1:
            self.calls += 1              # every pass starts on the same buffer parity (graphs freeze it)
