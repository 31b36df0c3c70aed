"""Per-request sampling parameters (the OpenAI / Anthropic request fields that reach the
sampler). Role of ``crates/sampling/src/lib.rs:54-103`` (``SamplingParams``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional


@dataclass
class SamplingParams:
    max_tokens: int = 256
    min_tokens: int = 0
    temperature: float = 0.0            # 0 -> greedy
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    top_n_sigma: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    # DRY ("don't repeat yourself"): a token that would extend a repeat of length n >= allowed_length
    # is penalised by multiplier * base ** (n - allowed_length); 0 multiplier = off
    dry_multiplier: float = 0.0
    dry_base: float = 1.75
    dry_allowed_length: int = 2
    dry_window: int = 1024
    # LZ-style loop guard: penalise the continuation of the longest earlier match of the current
    # suffix by lz_penalty * match_length (0 = off)
    lz_penalty: float = 0.0
    logit_bias: Dict[int, float] = field(default_factory=dict)
    seed: Optional[int] = None
    stop: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    logprobs: bool = False
    images: Optional[list] = None              # images of the request (data: URLs, bytes, arrays) for engines with a vision tower
    top_logprobs: int = 0
    n: int = 1
    timeout_s: float = 0.0
    grammar: Optional[object] = None    # constrained decoding matcher (server/grammar.py)
    adapter: Optional[str] = None       # LoRA adapter name (engine.load_adapter)
    # reasoning budget: once `thinking_budget` output tokens passed without the closing marker
    # `think_end_ids`, the sampler forces that marker token by token (0 = no limit)
    prediction_ids: List[int] = field(default_factory=list)   # predicted output (OpenAI `prediction`): used as drafts
    adaptive: Optional[object] = None   # sampling.adaptive.AdaptiveSampling: per-token temperature
    thinking_budget: int = 0
    think_end_ids: List[int] = field(default_factory=list)

    @property
    def greedy(self) -> bool:
        return not self.temperature > 0.0

    @property
    def needs_host_logits(self) -> bool:
        """True when plain device argmax / device sampling cannot serve the request."""
        return (bool(self.logit_bias) or self.top_n_sigma > 0 or self.grammar is not None or self.top_logprobs > 0
                or self.dry_multiplier > 0 or self.lz_penalty > 0
                or (self.thinking_budget > 0 and bool(self.think_end_ids)) or self.adaptive is not None)

    @property
    def has_penalties(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0)

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        if not 0 <= self.min_p <= 1:
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be > 0")
