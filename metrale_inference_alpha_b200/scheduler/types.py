"""Scheduler I/O contract: requests, sequences, step plans and results.

The scheduler core is pure host logic that talks to the device through an ``Executor``
(``execute(plan) -> StepResult``); tests drive it with a scripted executor, serving drives
it with the model runner. Role of the reference's ``crates/scheduler`` (``StepPlan``,
``Readback``, ``Effect``, ``DeviceIo``, ``ScriptedDeviceIo`` with ``Fault::{KvExhausted,Fatal}``).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..sampling.params import SamplingParams


class SeqStatus(enum.Enum):
    WAITING = 0
    PREFILL = 1
    DECODE = 2
    FINISHED = 3
    PREEMPTED = 4
    SWAPPED = 5


class FinishReason(str, enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"
    TIMEOUT = "timeout"
    ERROR = "error"


@dataclass
class Request:
    request_id: str
    prompt_ids: List[int]
    params: SamplingParams
    arrival: float = field(default_factory=time.monotonic)
    adapter: Optional[str] = None
    eos_token_id: Optional[int] = None
    mm: Optional[object] = None          # engine.multimodal.MultiModalInputs of a request with images

    @property
    def cache_ns(self):
        """Namespace of this request in the prefix cache: placeholder tokens of different images are the
        same ids, so cached blocks are only shared between requests that carry the same images."""
        return self.adapter if self.mm is None else (self.adapter, self.mm.digest)


class Sequence:
    def __init__(self, req: Request, seq_id: int):
        self.req = req
        self.seq_id = seq_id
        self.tokens: List[int] = list(req.prompt_ids)
        self.prompt_len = len(req.prompt_ids)
        self.num_computed = 0           # tokens whose KV / state is in the caches
        self.blocks: List[int] = []
        self.state_slot = 0
        self.status = SeqStatus.WAITING
        self.finish: Optional[FinishReason] = None
        self.cached_tokens = 0
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.logprobs: List[float] = []
        self.drafts: List[int] = []      # pending speculative tokens (not yet verified)
        self.draft_hidden = None         # target hidden row the drafter continues from
        self.accepted_draft_tokens = 0
        self.rejected_draft_tokens = 0
        self.spec_steps = 0
        self.sample_step = 0
        self.emitted = 0                 # output tokens already reported to the client
        self.stop_hit: Optional[str] = None
        self.swap_file: Optional[str] = None

    @property
    def output_ids(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def num_output(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def remaining_prefill(self) -> int:
        return max(0, len(self.tokens) - self.num_computed - (0 if self.status != SeqStatus.DECODE else 0))

    def is_finished(self) -> bool:
        return self.status == SeqStatus.FINISHED


@dataclass
class SeqStep:
    """One sequence's share of a step: feed `tokens` starting at position `start_pos`."""
    seq: Sequence
    tokens: List[int]
    start_pos: int
    sample: bool = True          # produce a token from the last row
    verify: int = 0              # number of trailing draft tokens (rows that need logits)


@dataclass
class StepPlan:
    kind: str                    # "prefill" | "decode" | "mixed" | "verify"
    items: List[SeqStep]
    num_tokens: int = 0

    def __post_init__(self):
        self.num_tokens = sum(len(i.tokens) for i in self.items)


@dataclass
class StepResult:
    """Per item: sampled token ids (one, or verify+1 for speculative rows) and log-probs."""
    tokens: List[List[int]]
    logprobs: Optional[List[List[float]]] = None
    hidden: Optional[object] = None      # device tensor of the sampled rows' hidden states
    device_ms: float = 0.0


class KvExhausted(RuntimeError):
    """The executor could not find KV blocks for the step (scheduler preempts and retries)."""


class FatalDeviceError(RuntimeError):
    """The device context is lost; the engine latches the fault and refuses new work."""


@dataclass
class RequestOutput:
    request_id: str
    new_token_ids: List[int]
    output_ids: List[int]              # all generated ids once `finished`; the new ids of this step before
    finished: bool
    finish_reason: Optional[str] = None
    prompt_tokens: int = 0
    cached_tokens: int = 0
    ttft_ms: Optional[float] = None
    decode_ms: Optional[float] = None
    logprobs: Optional[List[float]] = None
    accepted_draft_tokens: int = 0
    rejected_draft_tokens: int = 0
