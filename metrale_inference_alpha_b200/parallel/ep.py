"""Expert parallelism with token dispatch: instead of every rank running every token through its
local experts and all-reducing ``[tokens, hidden]`` (the reference's masked-local scheme, kept as
``EpMaskedAllReduce``-style fallback in ``models/moe.py``), each (token, expert) pair travels to
the rank that owns the expert, is processed there by the grouped tcgen05 expert GEMMs, and its
output travels back into the slot it was sent from, where the source rank applies the routing
weights. Both directions are ``ops/csrc/ep_a2a.cu``: 16-byte peer stores into symmetric-memory
landing zones, per-source counts and sequence-numbered flags (release / bounded acquire), double
buffered by parity; no NCCL call and no host synchronisation, and the sequence number is read
from device memory, so the layer stays inside CUDA graphs.

World size 1 runs the same kernels against the rank's own zone (the single-GPU test).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import _native

_VP8 = C.c_void_p * 8


class A2aArgs(C.Structure):
    _fields_ = [("rows", C.c_void_p), ("row_ld", C.c_longlong), ("n", C.c_int), ("row_bytes", C.c_int),
                ("dst_rank", C.c_void_p), ("dst_slot", C.c_void_p), ("meta", C.c_void_p), ("send_count", C.c_void_p),
                ("world", C.c_int), ("rank", C.c_int), ("capacity", C.c_int),
                ("zone", _VP8), ("zone_meta", _VP8), ("zone_count", _VP8), ("flag", _VP8),
                ("seq", C.c_uint), ("done", C.c_void_p), ("status", C.c_void_p), ("seq_ptr", C.c_void_p)]


_native.register_optional("mb_a2a_scatter", [C.POINTER(A2aArgs), C.c_void_p])
_native.register_optional("mb_a2a_wait", [C.c_void_p, C.c_int, C.c_uint, C.c_void_p, C.c_void_p])
_native.register_optional("mb_a2a_wait_dev", [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p])


class EpAllToAll:
    """Landing zones and protocol state of one expert-parallel group."""

    def __init__(self, rank: int, world: int, device, hidden: int, max_tokens: int, top_k: int, group=None):
        assert 1 <= world <= 8
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.H, self.K = hidden, top_k
        self.capacity = max_tokens * top_k                       # worst case: all of a rank's pairs go to one peer
        cap_rows = world * self.capacity
        self.x_bytes = cap_rows * hidden * 2                     # dispatched rows, bf16
        self.y_bytes = cap_rows * hidden * 2                     # returned rows, bf16
        # per parity: [x zone | y zone | x meta | x counts | y counts | x flags | y flags]
        self.meta_bytes = cap_rows * 4
        self.ctl_bytes = 4 * world * 4
        self.par_bytes = (self.x_bytes + self.y_bytes + self.meta_bytes + self.ctl_bytes + 255) // 256 * 256
        total = 2 * self.par_bytes + 256
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, group=group if group is not None else dist.group.WORLD)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            torch.cuda.synchronize(self.device)
            dist.barrier(group=group)
        else:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.ptrs = [self.buf.data_ptr()]
        self.done = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.seq = 0
        # the sequence number the kernels publish and wait for lives on the device and is advanced
        # by a device op, so that a replayed CUDA graph sees the current step's value; the host
        # copy only chooses the parity of the landing zones at launch (fixed per call site in a graph)
        self.seq_dev = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ layout helpers
    def _off(self, parity: int, what: str) -> int:
        base = parity * self.par_bytes
        o = {"x": 0, "y": self.x_bytes, "meta": self.x_bytes + self.y_bytes}
        if what in o:
            return base + o[what]
        c = base + self.x_bytes + self.y_bytes + self.meta_bytes
        return c + {"xcnt": 0, "ycnt": 1, "xflag": 2, "yflag": 3}[what] * self.world * 4

    def _local(self, parity: int, what: str, dtype, numel: int) -> torch.Tensor:
        o = self._off(parity, what)
        return self.buf[o:o + numel * torch.tensor([], dtype=dtype).element_size()].view(dtype)

    def _scatter(self, rows: torch.Tensor, dst_rank, dst_slot, meta, send_count, parity: int, which: str,
                 capacity: Optional[int] = None) -> None:
        from ..ops import _count, _ptr, _stream, runtime
        a = A2aArgs()
        a.rows, a.row_ld, a.n, a.row_bytes = _ptr(rows), rows.stride(0) * rows.element_size(), rows.shape[0], self.H * 2
        a.dst_rank, a.dst_slot, a.meta, a.send_count = _ptr(dst_rank), _ptr(dst_slot), _ptr(meta), _ptr(send_count)
        a.world, a.rank, a.capacity, a.seq = self.world, self.rank, capacity or self.capacity, self.seq
        a.seq_ptr = _ptr(self.seq_dev)
        zone, cnt, flag = ("x", "xcnt", "xflag") if which == "x" else ("y", "ycnt", "yflag")
        for r in range(self.world):
            a.zone[r] = self.ptrs[r] + self._off(parity, zone)
            a.zone_meta[r] = self.ptrs[r] + self._off(parity, "meta")
            a.zone_count[r] = self.ptrs[r] + self._off(parity, cnt)
            a.flag[r] = self.ptrs[r] + self._off(parity, flag)
        a.done = _ptr(self.done[0:1] if which == "x" else self.done[1:2])
        a.status = _ptr(runtime(self.device).status)
        _native.check(_native.lib().mb_a2a_scatter(C.byref(a), _stream()), "a2a_scatter")
        _count()

    def _wait(self, parity: int, which: str) -> None:
        from ..ops import _count, _ptr, _stream, runtime
        flags = self.ptrs[self.rank] + self._off(parity, "xflag" if which == "x" else "yflag")
        _native.check(_native.lib().mb_a2a_wait_dev(flags, self.world, _ptr(self.seq_dev),
                                                    _ptr(runtime(self.device).status), _stream()), "a2a_wait")
        _count()

    # ------------------------------------------------------------------ the MoE exchange
    def moe(self, x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, experts_per_rank: int, expert_fn,
            cap: Optional[int] = None):
        """x [T, H] bf16, routing weights / expert ids [T, K]. `expert_fn(rows bf16 [N, H], expert ids
        int32 [N, 1] (-1 = empty slot)) -> fp32 [N, H]` runs the local experts on received rows.
        Returns fp32 [T, H] = sum_j weights[t, j] * expert_{idx[t, j]}(x[t]).
        `cap`: rows each source may send in THIS call (the same number on every rank: the step's token
        count is known to all of them). The landing zones are then strided by it instead of by the
        allocation-time capacity, so the local experts run over about as many rows as were routed
        here, not over the whole capacity (a decode step sends tens of rows, the capacity is
        sized for a prefill chunk)."""
        T, K, W = x.shape[0], idx.shape[1], self.world
        Cp = self.capacity if cap is None else max(1, min(int(cap), self.capacity))
        assert T * K <= Cp and x.dtype == torch.bfloat16 and x.shape[1] == self.H
        self.seq += 1
        self.seq_dev.add_(1)
        parity = self.seq & 1
        dev = x.device
        # ---- where every (token, k) pair goes: destination rank and its slot in my region there
        flat = idx.reshape(-1).to(torch.int64)
        live = flat >= 0
        dest = torch.div(flat.clamp(min=0), experts_per_rank, rounding_mode="floor").clamp(0, W - 1)
        onehot = torch.nn.functional.one_hot(dest, W).to(torch.int32) * live[:, None].to(torch.int32)   # [T*K, W]
        slot = (torch.cumsum(onehot, 0) - 1).gather(1, dest[:, None]).squeeze(1).clamp(min=0).to(torch.int32)
        send_count = onehot.sum(0).to(torch.int32)
        dest32 = torch.where(live, dest, torch.full_like(dest, -1)).to(torch.int32)
        rows = x.repeat_interleave(K, 0) if K > 1 else x                              # pair p = token p // K
        self._scatter(rows, dest32, slot, flat.to(torch.int32), send_count, parity, "x", Cp)
        self._wait(parity, "x")
        # ---- local experts over everything that landed here
        n_cap = W * Cp
        xz = self._local(parity, "x", torch.bfloat16, n_cap * self.H).view(n_cap, self.H)
        meta = self._local(parity, "meta", torch.int32, n_cap).view(W, Cp)
        rcnt = self._local(parity, "xcnt", torch.int32, W)
        valid = torch.arange(Cp, device=dev, dtype=torch.int32)[None, :] < rcnt[:, None]
        eids = torch.where(valid, meta, torch.full_like(meta, -1)).reshape(n_cap, 1)
        y = expert_fn(xz, eids)                                                       # fp32 [n_cap, H]
        # ---- every landed row goes back to its source, into the slot it came from
        back_rank = torch.where(valid, torch.arange(W, device=dev, dtype=torch.int32)[:, None].expand(W, Cp),
                                torch.full_like(meta, -1)).reshape(-1).contiguous()
        back_slot = torch.arange(Cp, device=dev, dtype=torch.int32).repeat(W)
        self._scatter(y.to(torch.bfloat16), back_rank, back_slot, None, rcnt, parity, "y", Cp)
        self._wait(parity, "y")
        yz = self._local(parity, "y", torch.bfloat16, n_cap * self.H).view(n_cap, self.H)
        # ---- combine: pair p's result sits in my y zone at (dest[p], slot[p])
        pos = dest * Cp + slot.to(torch.int64)
        got = yz.index_select(0, pos).view(T, K, self.H).float()
        got = torch.where(live.view(T, K, 1), got, torch.zeros_like(got))
        return (got * weights.view(T, K, 1).float()).sum(1)

    # ------------------------------------------------------------------ hook used by models/moe.py
    def dispatch_compute_combine(self, dec, a, weights: torch.Tensor, idx: torch.Tensor, w) -> torch.Tensor:
        """Routed-expert output for all T tokens, fp32 [T, H], to be summed over ranks by the caller.
        Activations are replicated in this engine, so each rank dispatches only its slice of the
        tokens (the others' rows stay zero here and arrive through the caller's sum over ranks)."""
        from ..models.moe import routed_experts
        T = a.M
        per = (T + self.world - 1) // self.world
        lo, hi = min(T, self.rank * per), min(T, (self.rank + 1) * per)
        xb = a.bf16 if a.bf16 is not None else a.data
        fmt = a.fmt
        E_local = len(w.experts) if w.experts else w.grouped.num

        def expert_fn(rows, eids):
            ar = dec._as_act(rows, fmt)
            ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
            return routed_experts(dec, ar, ones, eids, w)
        out = torch.zeros(T, self.H, dtype=torch.float32, device=xb.device)
        cap = per * idx.shape[1]                      # every rank derives the same bound from the step's token count
        if hi > lo:
            out[lo:hi] = self.moe(xb[lo:hi].contiguous(), weights[lo:hi].contiguous(), idx[lo:hi].contiguous(),
                                  E_local, expert_fn, cap=cap)
        else:
            # nothing to send, but the peers still wait for this rank's flags and rows for its experts
            dummy_x = torch.zeros(1, self.H, dtype=torch.bfloat16, device=xb.device)
            self.moe(dummy_x, torch.zeros(1, idx.shape[1], device=xb.device),
                     torch.full((1, idx.shape[1]), -1, dtype=idx.dtype, device=xb.device), E_local, expert_fn, cap=cap)
        return out
