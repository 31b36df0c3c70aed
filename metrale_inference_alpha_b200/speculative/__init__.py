"""Speculative-decoding policy (host code): the MTP throughput gate, the draft-width ladder,
adaptive rung, n-gram prompt lookup, DFlash width resolver, D-Cut pruning.
Role of the reference's ``crates/speculative`` and ``crates/model-layers/src/speculative/ladder.rs``."""
from .gate import MtpGate, SpecStats  # noqa: F401
from .ladder import KLadder, AdaptiveRung, DflashRung, spec_capacity, dcut_plan  # noqa: F401
from .ngram import NgramProposer  # noqa: F401
