"""Scheduling policies: FIFO (prefill as soon as there is work) and a time-between-tokens
deadline policy that bounds how long running decodes may wait behind prefill chunks.
Role of ``crates/server/src/scheduler/scheduling_policy.rs:56-153``."""
from __future__ import annotations

import time
from dataclasses import dataclass


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 128              # batch cap
    max_prefill_tokens: int = 8192       # per-step prefill token budget (chunked prefill)
    max_model_len: int = 32768
    block_size: int = 16
    policy: str = "fifo"                 # fifo | tbt | slai
    tbt_deadline_ms: float = 100.0
    decode_reserve_tokens: int = 256     # admission watermark: prompt + min(max_tokens, this)
    enable_prefix_caching: bool = True
    mixed_prefill_decode: bool = False   # run decode rows and a prefill chunk in one forward
    request_timeout_s: float = 300.0
    preempt_mode: str = "recompute"      # recompute | swap
    batch_rungs: tuple = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128)
    decode_ring_slots: int = 0           # recurrent models: state snapshots kept per decoding sequence for rollback (0 = off)
    decode_ring_interval: int = 16       # a snapshot every this many generated tokens ...
    decode_ring_boundary_tokens: tuple = ()   # ... and whenever one of these token ids is generated


class FifoPolicy:
    def should_prefill(self, have_prefill: bool, have_decode: bool, now: float) -> bool:
        return have_prefill

    def prefill_budget(self, cfg: SchedulerConfig, have_decode: bool) -> int:
        return cfg.max_prefill_tokens

    def note_decode(self, now: float) -> None:
        pass


class TbtDeadlinePolicy:
    """Interleave: once running sequences have waited `tbt_deadline_ms` since their last
    decode step, decode goes first; prefill chunks shrink while decodes are waiting."""

    def __init__(self, deadline_ms: float):
        self.deadline = deadline_ms / 1e3
        self.last_decode = time.monotonic()

    def should_prefill(self, have_prefill: bool, have_decode: bool, now: float) -> bool:
        if not have_prefill:
            return False
        if not have_decode:
            return True
        return (now - self.last_decode) < self.deadline

    def prefill_budget(self, cfg: SchedulerConfig, have_decode: bool) -> int:
        return max(256, cfg.max_prefill_tokens // 4) if have_decode else cfg.max_prefill_tokens

    def note_decode(self, now: float) -> None:
        self.last_decode = now


class SlaiPolicy:
    """Deadline-aware scheduling (the reference's `--scheduler slai`,
    ``crates/server/src/scheduling_policy.rs:69-153``): no prefill is started while the running
    decodes have waited 80 % of the time-between-tokens deadline since their last token; prefill
    chunks are never shrunk (a smaller slice does not shorten the step, it only slows the prefill);
    admission takes the front of the queue first, then the shortest prompts, so that short requests
    overtake long ones but the head of the line can never starve."""

    def __init__(self, deadline_ms: float):
        self.deadline = deadline_ms / 1e3
        self.last_decode = time.monotonic()

    def should_prefill(self, have_prefill: bool, have_decode: bool, now: float) -> bool:
        if not have_prefill:
            return False
        if not have_decode:
            return True
        return (now - self.last_decode) < 0.8 * self.deadline

    def prefill_budget(self, cfg: SchedulerConfig, have_decode: bool) -> int:
        return cfg.max_prefill_tokens

    def note_decode(self, now: float) -> None:
        self.last_decode = now

    @staticmethod
    def order_waiting(waiting) -> None:
        """In place: seat 0 stays, the rest are ordered by prompt length (stable)."""
        if len(waiting) > 2:
            head = waiting.popleft()
            rest = sorted(waiting, key=lambda s: len(s.tokens))
            waiting.clear()
            waiting.append(head)
            waiting.extend(rest)


def make_policy(cfg: SchedulerConfig):
    if cfg.policy == "tbt":
        return TbtDeadlinePolicy(cfg.tbt_deadline_ms)
    if cfg.policy == "slai":
        return SlaiPolicy(cfg.tbt_deadline_ms)
    if cfg.policy != "fifo":
        raise ValueError(f"unknown scheduler policy {cfg.policy!r} (fifo | tbt | slai)")
    return FifoPolicy()
