"""Adaptive sampling (`--adaptive-sampling`): the temperature of every token follows what the
model is generating and how it has been behaving.

* zone: a tool call caps the temperature at 0.3, grammar-constrained output scales it by 0.6,
  reasoning and free text keep the request's value (tool call wins over reasoning, reasoning over
  grammar);
* greedy gate: when the top-1 probability reaches the zone's threshold (0.8 tool call, 0.85
  structured, 0.9 free text, 0.95 reasoning) the token is taken greedily;
* entropy boost: after 8 / 16 / 32 consecutive tokens with entropy below 0.5 nats the temperature
  rises by 0.1 / 0.2 / 0.3 (never inside a tool call);
* repetition multiplier: the share of distinct 3..6-byte windows over the little-endian bytes of
  the last 128 output tokens, recomputed every 16 tokens once there are 32; below 0.35 / 0.25 /
  0.15 the temperature is multiplied by 1.2 / 1.4 / 1.8 (never inside a tool call).

A request temperature of 0 always stays 0. Role of the reference's
``crates/server/src/adaptive_sampler.rs``.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

FREE, THINKING, TOOL_CALL, STRUCTURED = "free_text", "thinking", "tool_call", "structured"
_GATE = {TOOL_CALL: 0.8, STRUCTURED: 0.85, FREE: 0.9, THINKING: 0.95}


def _find_last(hay: Sequence[int], needle: Sequence[int]) -> int:
    n = len(needle)
    if n == 0:
        return -1
    for i in range(len(hay) - n, -1, -1):
        if list(hay[i:i + n]) == list(needle):
            return i
    return -1


@dataclass
class AdaptiveSampling:
    base_temperature: float
    think_end_ids: List[int] = field(default_factory=list)     # reasoning is open until this appears
    thinking_open: bool = False
    tool_open_ids: List[int] = field(default_factory=list)
    tool_close_ids: List[int] = field(default_factory=list)
    zone: str = FREE
    low_entropy_run: int = 0
    lz_ratio: float = 1.0
    _lz_checked_at: int = 0

    # ---- state updates
    def update_zone(self, output_tokens: Sequence[int], grammar_active: bool) -> str:
        tool = False
        if self.tool_open_ids:
            o = _find_last(output_tokens, self.tool_open_ids)
            tool = o >= 0 and _find_last(output_tokens, self.tool_close_ids) < o
        thinking = self.thinking_open and self.think_end_ids and _find_last(output_tokens, self.think_end_ids) < 0
        self.zone = TOOL_CALL if tool else THINKING if thinking else STRUCTURED if grammar_active else FREE
        return self.zone

    def observe(self, logits: torch.Tensor) -> None:
        """Entropy (nats) of the distribution the token was drawn from extends or resets the run."""
        x = logits.float()
        m = x.max()
        if not torch.isfinite(m):
            return
        p = torch.softmax(x - m, -1)
        ent = float(-(p * torch.log(p.clamp_min(1e-10))).sum())
        self.low_entropy_run = self.low_entropy_run + 1 if ent < 0.5 else 0

    def update_repetition(self, output_tokens: Sequence[int]) -> None:
        n = len(output_tokens)
        if n < 32 or n - self._lz_checked_at < 16:
            return
        self._lz_checked_at = n
        data = b"".join(struct.pack("<I", t & 0xFFFFFFFF) for t in output_tokens[-128:])
        seen, total = set(), 0
        for w in range(3, 7):
            for i in range(len(data) - w + 1):
                seen.add(data[i:i + w])
                total += 1
        self.lz_ratio = len(seen) / total if total else 1.0

    # ---- decisions
    def temperature(self) -> float:
        base = self.base_temperature
        if base == 0.0:
            return 0.0
        t = min(base, 0.3) if self.zone == TOOL_CALL else base * 0.6 if self.zone == STRUCTURED else base
        if self.zone == TOOL_CALL:
            return t
        run = self.low_entropy_run
        boost = 0.0 if run < 8 else 0.1 if run < 16 else 0.2 if run < 32 else 0.3
        r = self.lz_ratio
        mult = 1.8 if r < 0.15 else 1.4 if r < 0.25 else 1.2 if r < 0.35 else 1.0
        return (t + boost) * mult

    def greedy(self, logits: torch.Tensor) -> bool:
        if self.base_temperature == 0.0:
            return True
        x = logits.float()
        m = x.max()
        if not torch.isfinite(m):
            return False
        top = 1.0 / float(torch.exp(x - m).sum())
        return top >= _GATE[self.zone]

    def step(self, logits: torch.Tensor, output_tokens: Sequence[int], grammar_active: bool) -> float:
        """Temperature for the token about to be sampled from `logits` (0 = greedy)."""
        self.update_zone(output_tokens, grammar_active)
        self.update_repetition(output_tokens)
        t = 0.0 if self.greedy(logits) else self.temperature()
        self.observe(logits)
        return t
