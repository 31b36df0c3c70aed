"""Continuous-batching scheduler core (host logic only).

Each ``plan()`` call does: time-outs -> admission (KV reservation ``prompt + min(max_tokens,
watermark)``, stop at the first misfit, forced-oversize liveness) -> pick a lane (prefill
chunk(s), decode, or a mixed step) according to the policy. ``apply()`` folds the executor's
result back: append tokens, accept / reject speculative drafts, stop conditions, retire
finished sequences (publishing their blocks to the prefix cache), state snapshots for
recurrent models. KV exhaustion is answered by evicting prefix-cache blocks, then by
preempting the most recently admitted running sequence (requeue for re-prefill, or spill).
Role of the reference's ``crates/server/src/scheduler`` (``core/tick.rs``, ``admission.rs``,
``phase_start_prefills.rs``, ``phase_continue_prefills.rs``, ``core/lane_decode.rs``,
``preempt.rs``, ``core/end_tick.rs``).
"""
from __future__ import annotations

import itertools
import time
from collections import deque
from typing import Callable, Deque, Dict, List, Optional

from ..cache import BlockAllocator, NoFreeBlocks, RadixTree
from .policy import SchedulerConfig, make_policy
from .types import (FinishReason, Request, RequestOutput, SeqStatus, SeqStep, Sequence, StepPlan,
                    StepResult)


class SchedulerCore:
    def __init__(self, cfg: SchedulerConfig, allocator: BlockAllocator, prefix: Optional[RadixTree] = None,
                 state_pool=None, clock: Callable[[], float] = time.monotonic, spill=None):
        self.cfg = cfg
        self.alloc = allocator
        self.prefix = prefix if cfg.enable_prefix_caching else None
        self.pool = state_pool
        self.clock = clock
        self.spill = spill
        self.policy = make_policy(cfg)
        self.waiting: Deque[Sequence] = deque()
        self.prefilling: List[Sequence] = []
        self.running: List[Sequence] = []
        self.swapped: Deque[Sequence] = deque()
        self._ids = itertools.count(1)
        self._by_req: Dict[str, Sequence] = {}
        self._finished_now: List[Sequence] = []
        self.snapshot_interval = 256
        self.stats = {"admitted": 0, "preempted": 0, "finished": 0, "prefill_tokens": 0, "decode_tokens": 0,
                      "steps": 0, "evicted_blocks": 0, "timeouts": 0}

    # ------------------------------------------------------------------ intake
    def add_request(self, req: Request) -> Sequence:
        req.params.validate()
        if len(req.prompt_ids) == 0:
            raise ValueError("empty prompt")
        if len(req.prompt_ids) >= self.cfg.max_model_len:
            raise ValueError(f"prompt of {len(req.prompt_ids)} tokens exceeds max_model_len {self.cfg.max_model_len}")
        seq = Sequence(req, next(self._ids))
        self.waiting.append(seq)
        self._by_req[req.request_id] = seq
        return seq

    def abort(self, request_id: str) -> bool:
        seq = self._by_req.get(request_id)
        if seq is None or seq.is_finished():
            return False
        self._finish(seq, FinishReason.ABORT, publish=False)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running or self.swapped)

    @property
    def num_active(self) -> int:
        return len(self.prefilling) + len(self.running)

    # ------------------------------------------------------------------ block bookkeeping
    def _blocks_for(self, tokens: int) -> int:
        return (tokens + self.cfg.block_size - 1) // self.cfg.block_size

    def _free_capacity(self) -> int:
        return self.alloc.num_free + (self.prefix.evictable_blocks() if self.prefix else 0)

    def _alloc_blocks(self, n: int) -> List[int]:
        if n <= 0:
            return []
        if self.alloc.num_free < n and self.prefix:
            self.stats["evicted_blocks"] += self.prefix.evict(n - self.alloc.num_free)
        return self.alloc.alloc(n)

    def _ensure_blocks(self, seq: Sequence, upto_tokens: int) -> None:
        need = self._blocks_for(upto_tokens) - len(seq.blocks)
        if need > 0:
            seq.blocks += self._alloc_blocks(need)

    # ------------------------------------------------------------------ admission
    def _admit(self) -> None:
        cfg = self.cfg
        while self.swapped and self.num_active < cfg.max_num_seqs:
            seq = self.swapped[0]
            if self._free_capacity() < self._blocks_for(len(seq.tokens) + 1):
                break
            self.swapped.popleft()
            self.spill.restore(seq, self)
            (self.running if seq.num_computed >= len(seq.tokens) - 1 else self.prefilling).append(seq)
            seq.status = SeqStatus.DECODE if seq in self.running else SeqStatus.PREFILL
        order = getattr(self.policy, "order_waiting", None)
        if order is not None:
            order(self.waiting)
        while self.waiting and self.num_active < cfg.max_num_seqs:
            seq = self.waiting[0]
            if seq.is_finished():
                self.waiting.popleft()
                continue
            matched, snap = [], None
            if self.prefix is not None and seq.num_computed == 0:
                m = self.prefix.match(seq.tokens, seq.req.cache_ns)
                matched, snap = m.blocks, m.snapshot
            reserve = min(seq.req.params.max_tokens, cfg.decode_reserve_tokens)
            need = self._blocks_for(len(seq.tokens) + reserve) - len(matched)
            if self._free_capacity() < need:
                self.alloc.free(matched)
                total = self.alloc.num_blocks - 1
                if self.num_active == 0 and self._blocks_for(len(seq.tokens) + 1) > total:
                    # can never fit: fail it rather than block the queue forever
                    self.waiting.popleft()
                    self._finish(seq, FinishReason.ERROR, publish=False)
                    continue
                if self.num_active == 0 and self._blocks_for(len(seq.tokens) + 1) <= self._free_capacity():
                    # forced-oversize liveness: admit with a smaller reserve when alone
                    if self.prefix is not None and seq.num_computed == 0:
                        m = self.prefix.match(seq.tokens, seq.req.cache_ns)
                        matched, snap = m.blocks, m.snapshot
                else:
                    break                                   # stop at the first misfit (FIFO)
            self.waiting.popleft()
            seq.blocks = list(matched)
            seq.cached_tokens = len(matched) * cfg.block_size
            seq.num_computed = seq.cached_tokens
            if self.pool is not None:
                seq.state_slot = self.pool.alloc()
                if snap is not None:
                    self.pool.restore(snap, seq.state_slot)
            try:
                self._ensure_blocks(seq, len(seq.tokens))
            except NoFreeBlocks:
                self._release(seq)
                self.waiting.appendleft(seq)
                break
            seq.status = SeqStatus.PREFILL
            self.prefilling.append(seq)
            self.stats["admitted"] += 1

    # ------------------------------------------------------------------ preemption
    def preempt_one(self, exclude: Optional[Sequence] = None) -> Optional[Sequence]:
        """Evict the most recently admitted running (else prefilling) sequence."""
        pool = [s for s in self.running if s is not exclude] or [s for s in self.prefilling if s is not exclude]
        if not pool:
            return None
        victim = max(pool, key=lambda s: s.seq_id)
        (self.running if victim in self.running else self.prefilling).remove(victim)
        self.stats["preempted"] += 1
        if self.cfg.preempt_mode == "swap" and self.spill is not None and self.spill.save(victim, self):
            victim.status = SeqStatus.SWAPPED
            self.swapped.append(victim)
        else:
            self._release(victim)
            victim.num_computed = 0
            victim.cached_tokens = 0
            victim.drafts = []
            victim.status = SeqStatus.WAITING
            self.waiting.appendleft(victim)
        return victim

    def _release(self, seq: Sequence) -> None:
        self.alloc.free(seq.blocks)
        seq.blocks = []
        ring = getattr(seq, "decode_ring", None)
        if ring is not None and self.pool is not None:
            for sid in ring.clear():
                self.pool.release_snapshot(sid)
        if self.pool is not None and seq.state_slot:
            self.pool.free(seq.state_slot)
            seq.state_slot = 0

    # ------------------------------------------------------------------ planning
    def plan(self) -> Optional[StepPlan]:
        now = self.clock()
        self._check_timeouts(now)
        self._admit()
        have_prefill, have_decode = bool(self.prefilling), bool(self.running)
        if not (have_prefill or have_decode):
            return None
        if self.policy.should_prefill(have_prefill, have_decode, now):
            items = self._prefill_items(self.policy.prefill_budget(self.cfg, have_decode))
            if self.cfg.mixed_prefill_decode and have_decode:
                dec = self._decode_items()
                # growing a decode sequence can preempt a prefilling one when the pool is
                # exhausted: its blocks are gone, so its chunk leaves the plan too
                items = dec + [i for i in items if i.seq in self.prefilling]
                return StepPlan("mixed", items) if items else None
            if items:
                return StepPlan("prefill", items)
        items = self._decode_items()
        if not items:
            return None
        self.policy.note_decode(now)
        return StepPlan("verify" if any(i.verify for i in items) else "decode", items)

    def plan_ahead(self, plan: StepPlan) -> Optional[StepPlan]:
        """The decode step that follows `plan`, planned before `plan`'s tokens are known (one step
        of look-ahead: the device feeds each sampled token straight into the next step, so the
        engine can launch step t + 1 while it reads back step t). Every sequence advances by one
        position; the token values are placeholders (-1). Returns None whenever the next step is
        not simply "the same sequences, one position later": something waits for admission, a
        sequence reaches its length limit at `plan`, or a block is missing (no preemption here).
        A sequence that ends at `plan` by a stop token still occupies its row in the look-ahead
        step; `apply` skips finished sequences, so that row's token is discarded.
        Role of the reference's one-step-ahead decode (``crates/server/src/scheduler/core/pipeline.rs:1-22,124-149``)."""
        if plan.kind != "decode" or self.waiting or self.prefilling or self.swapped:
            return None
        if len(plan.items) != len(self.running):
            return None
        items = []
        for it, seq in zip(plan.items, self.running):
            if it.seq is not seq or seq.is_finished() or seq.drafts or it.verify or len(it.tokens) != 1:
                return None
            L = len(seq.tokens)
            if seq.num_output + 2 > seq.req.params.max_tokens or L + 2 > self.cfg.max_model_len:
                return None
            if self._blocks_for(L + 1) > len(seq.blocks) and self._free_capacity() < 1:
                return None
            items.append(SeqStep(seq, [-1], L, sample=True))
        try:
            for it in items:
                self._ensure_blocks(it.seq, it.start_pos + 1)
        except NoFreeBlocks:
            return None
        return StepPlan("decode", items)

    def _prefill_items(self, budget: int) -> List[SeqStep]:
        items = []
        for seq in self.prefilling:
            if budget <= 0:
                break
            remaining = len(seq.tokens) - seq.num_computed
            n = min(remaining, budget)
            if n <= 0:
                continue
            start = seq.num_computed
            if (n == remaining and self.pool is not None and self.prefix is not None
                    and getattr(self.prefix, "needs_snapshot", False)):
                # recurrent models: a later request with the same prompt can only resume from a state
                # snapshot, and the longest reusable prefix ends at the last block boundary below the
                # prompt's end: stop this chunk there, so that the snapshot exists (the remaining
                # < one block of tokens runs as the next step)
                boundary = ((len(seq.tokens) - 1) // self.cfg.block_size) * self.cfg.block_size
                if start < boundary and boundary >= self.snapshot_interval:
                    n = boundary - start
            items.append(SeqStep(seq, seq.tokens[start:start + n], start, sample=(start + n == len(seq.tokens))))
            budget -= n
        return items

    def _decode_items(self) -> List[SeqStep]:
        items = []
        preempted = False                                   # membership is re-checked only after a preemption
        for seq in list(self.running):
            if preempted and seq not in self.running:
                continue                                    # preempted while planning
            drafts = seq.drafts
            feed = [seq.tokens[-1]] + drafts
            while True:
                try:
                    self._ensure_blocks(seq, len(seq.tokens) + len(drafts))
                    break
                except NoFreeBlocks:
                    victim = self.preempt_one(exclude=seq)
                    if victim is None:
                        # alone and out of blocks: the sequence ends here
                        self._finish(seq, FinishReason.LENGTH)
                        feed = None
                        break
                    preempted = True
                    items = [i for i in items if i.seq is not victim]
            if feed is None:
                continue
            items.append(SeqStep(seq, feed, len(seq.tokens) - 1, sample=True, verify=len(drafts)))
        return items

    # ------------------------------------------------------------------ results
    def apply(self, plan: StepPlan, result: StepResult, drafts: Optional[List[List[int]]] = None
              ) -> List[RequestOutput]:
        self.stats["steps"] += 1
        now = self.clock()
        touched: List[Sequence] = []
        for i, item in enumerate(plan.items):
            seq = item.seq
            if seq.is_finished():
                continue
            n_fed = len(item.tokens)
            if seq.status == SeqStatus.PREFILL:
                seq.num_computed = item.start_pos + n_fed
                self.stats["prefill_tokens"] += n_fed
                self._maybe_snapshot(seq)
                if not item.sample:
                    continue
                self.prefilling.remove(seq)
                self.running.append(seq)
                seq.status = SeqStatus.DECODE
                new = result.tokens[i][:1]
            elif item.verify:
                target = result.tokens[i]                   # verify + 1 target tokens
                n_acc = 0
                while n_acc < item.verify and item.tokens[1 + n_acc] == target[n_acc]:
                    n_acc += 1
                new = list(item.tokens[1:1 + n_acc]) + [target[n_acc]]
                seq.accepted_draft_tokens += n_acc
                seq.rejected_draft_tokens += item.verify - n_acc
                seq.spec_steps += 1
                seq.num_computed = item.start_pos + 1 + n_acc      # rewind over rejected rows
                seq.last_accept = n_acc
            else:
                new = result.tokens[i][:1]
                seq.num_computed = item.start_pos + 1
                seq.last_accept = 0
                self._ring_record(seq, new)
            seq.drafts = []
            if drafts is not None and i < len(drafts) and drafts[i]:
                seq.drafts = list(drafts[i])
            if result.logprobs is not None:
                seq.logprobs += list(result.logprobs[i][:len(new)])
            self._append_tokens(seq, new, now)
            touched.append(seq)
        outs = [self._output(s) for s in touched]
        outs += [self._output(s) for s in self._finished_now if s not in touched]
        self._finished_now = []
        return outs

    def _append_tokens(self, seq: Sequence, new: List[int], now: float) -> None:
        p = seq.req.params
        for t in new:
            seq.tokens.append(t)
            self.stats["decode_tokens"] += 1
            if seq.first_token_time is None:
                seq.first_token_time = now
            n_out = seq.num_output
            eos = seq.req.eos_token_id
            if n_out >= p.min_tokens and ((not p.ignore_eos and eos is not None and t == eos)
                                          or t in p.stop_token_ids):
                self._finish(seq, FinishReason.STOP)
                return
            if n_out >= p.max_tokens or len(seq.tokens) >= self.cfg.max_model_len:
                self._finish(seq, FinishReason.LENGTH)
                return

    def finish_with_stop(self, seq: Sequence, keep_output_tokens: int, stop: str) -> None:
        """Used by the engine when a stop *string* matched: truncate and retire."""
        del seq.tokens[seq.prompt_len + keep_output_tokens:]
        seq.stop_hit = stop
        self._finish(seq, FinishReason.STOP)

    # ------------------------------------------------------------------ decode rollback
    def _ring_record(self, seq: Sequence, new: List[int]) -> None:
        """After a plain decode step: the recurrent state now covers every token but the one just
        sampled, which is exactly what a rollback keeping `num_output + 1` tokens must resume from."""
        c = self.cfg
        if self.pool is None or c.decode_ring_slots <= 0 or not new:
            return
        pos = seq.num_output + 1                            # generated tokens once `new` is appended
        if pos % max(1, c.decode_ring_interval) != 0 and new[0] not in c.decode_ring_boundary_tokens:
            return
        ring = getattr(seq, "decode_ring", None)
        if ring is None:
            from .decode_ring import StateDecodeRing
            ring = seq.decode_ring = StateDecodeRing(c.decode_ring_slots)
        sid = self.pool.snapshot(seq.state_slot)
        if sid is None:
            return
        drop = ring.record(pos, sid)
        if drop is not None:
            self.pool.release_snapshot(drop)

    def rollback_positions(self, seq: Sequence) -> List[int]:
        """Output lengths this sequence can be rolled back to right now."""
        if self.pool is None:
            return list(range(1, seq.num_output + 1))
        ring = getattr(seq, "decode_ring", None)
        return [p for p in (ring.positions() if ring else []) if p <= seq.num_output]

    def rollback(self, seq: Sequence, keep_output_tokens: int) -> bool:
        """Truncate a decoding sequence to its first `keep_output_tokens` generated tokens and
        continue from there. Attention KV needs nothing (later slots are rewritten); a recurrent
        model needs the ring snapshot taken at exactly that length, else the rollback is declined
        (role of the reference's boundary rollback, ``crates/server/src/scheduler/rollback.rs`` with
        ``ssm_decode_ring.rs``)."""
        if seq.is_finished() or seq not in self.running or not (0 < keep_output_tokens <= seq.num_output):
            return False
        if keep_output_tokens == seq.num_output:
            return True
        if self.pool is not None:
            ring = getattr(seq, "decode_ring", None)
            e = ring.find(keep_output_tokens) if ring else None
            if e is None or not self.pool.available(e.snapshot):
                return False
            self.pool.restore(e.snapshot, seq.state_slot)
            for sid in ring.truncate_after(keep_output_tokens):
                self.pool.release_snapshot(sid)
        del seq.tokens[seq.prompt_len + keep_output_tokens:]
        if seq.logprobs:
            del seq.logprobs[keep_output_tokens:]
        seq.drafts = []
        seq.num_computed = len(seq.tokens) - 1
        self.stats["rollbacks"] = self.stats.get("rollbacks", 0) + 1
        return True

    def _maybe_snapshot(self, seq: Sequence) -> None:
        if self.pool is None or self.prefix is None or not self.prefix.needs_snapshot:
            return
        p = seq.num_computed
        if p % self.cfg.block_size == 0 and p >= self.snapshot_interval and p < len(seq.tokens):
            sid = self.pool.snapshot(seq.state_slot)
            if sid is not None:
                if not hasattr(seq, "snapshots"):
                    seq.snapshots = {}
                seq.snapshots[p] = sid

    def _finish(self, seq: Sequence, reason: FinishReason, publish: bool = True) -> None:
        if seq.is_finished():
            return
        for lst in (self.prefilling, self.running):
            if seq in lst:
                lst.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)
        if seq in self.swapped:
            self.swapped.remove(seq)
            if self.spill is not None and hasattr(self.spill, "drop"):
                self.spill.drop(seq)
        if publish and self.prefix is not None and seq.blocks:
            n_full = min(seq.num_computed, len(seq.tokens)) // self.cfg.block_size
            if n_full:
                self.prefix.insert(seq.tokens[:n_full * self.cfg.block_size], seq.blocks[:n_full],
                                   seq.req.cache_ns, getattr(seq, "snapshots", None))
        self._release(seq)
        seq.status = SeqStatus.FINISHED
        seq.finish = reason
        seq.finish_time = self.clock()
        seq.drafts = []
        self.stats["finished"] += 1
        self._finished_now.append(seq)

    def _check_timeouts(self, now: float) -> None:
        for seq in list(self.waiting) + list(self.prefilling) + list(self.running) + list(self.swapped):
            limit = seq.req.params.timeout_s or self.cfg.request_timeout_s
            if limit and now - seq.req.arrival > limit:
                self.stats["timeouts"] += 1
                self._finish(seq, FinishReason.TIMEOUT, publish=False)

    def _output(self, seq: Sequence) -> RequestOutput:
        new = seq.tokens[seq.prompt_len + seq.emitted:]
        seq.emitted = seq.num_output
        done = seq.is_finished()
        ttft = None if seq.first_token_time is None else (seq.first_token_time - seq.req.arrival) * 1e3
        dec = None
        if seq.finish_time is not None and seq.first_token_time is not None:
            dec = (seq.finish_time - seq.first_token_time) * 1e3
        # the cumulative ids travel with the final output only (a per-step copy would be quadratic)
        return RequestOutput(seq.req.request_id, new, seq.output_ids if done else new, done,
                             seq.finish.value if seq.finish else None, seq.prompt_len, seq.cached_tokens,
                             ttft, dec, seq.logprobs if seq.req.params.logprobs else None,
                             seq.accepted_draft_tokens, seq.rejected_draft_tokens)

    def drain_finished(self) -> List[RequestOutput]:
        outs = [self._output(s) for s in self._finished_now]
        self._finished_now = []
        return outs

    def snapshot(self) -> dict:
        """State summary for metrics and the speculative gate."""
        return {"waiting": len(self.waiting), "prefilling": len(self.prefilling), "running": len(self.running),
                "swapped": len(self.swapped), "free_blocks": self.alloc.num_free,
                "used_blocks": self.alloc.num_used, **self.stats}
