"""Kernel-resolution audit: which kernel launcher actually served each class of op.

The ops layer picks a kernel per call (tcgen05 or mma.sync attention, grouped or per-expert MoE, chunked or
sequential scans, fused or separate quantisers, W4A4 or W4A16 ...); a silent fall to a slower path is a
performance bug that no numerics test sees. While an audit is on, every successful launcher call is counted
by name. ``resolve(rules)`` maps op classes to the launchers that may serve them and reports, per class,
which ones ran and how often; ``require(...)`` turns an expectation ("prefill attention must run on
attn_prefill_tc") into a failure. Launches inside a replayed CUDA graph are not seen (they were counted when
the graph was captured).

Reference: ``crates/telemetry/src/kernel_audit.rs`` (kernel-resolution audit) beside the launch trace.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

from ..ops import _native

# op class -> launcher names (as passed to _native.check) that can serve it, fastest first
DEFAULT_RULES: Dict[str, List[str]] = {
    "gemm": ["gemm", "a16_gemv", "a16_dequant"],
    "prefill attention": ["attn_prefill_tc", "paged_attention"],
    "mla attention": ["mla_attention"],
    "row ops": ["row_op"],
    "rope + kv write": ["qk_norm_rope_kvwrite"],
    "moe routing": ["moe_route", "moe_route_shared"],
    "moe sort / gather / combine": ["moe_sort", "moe_gather", "moe_combine", "moe_finish"],
    "gated delta rule": ["gdn_chunked", "gdn_recurrence"],
    "kimi delta attention": ["kda_chunked", "kda_recurrence"],
    "mamba2 scan": ["mamba2_ssd", "mamba2_scan"],
    "causal conv": ["causal_conv1d_par", "causal_conv1d"],
    "sparse attention select": ["index_score", "topk_select", "gather_rows"],
    "sampling": ["argmax", "sample"],
}


class KernelAudit:
    def __init__(self):
        self.counts: Dict[str, int] = {}
        self._prev = None

    def __enter__(self) -> "KernelAudit":
        self._prev = _native._audit
        _native._audit = self.counts
        return self

    def __exit__(self, *exc) -> None:
        _native._audit = self._prev

    def resolve(self, rules: Optional[Dict[str, List[str]]] = None) -> Dict[str, Dict[str, int]]:
        """Per op class, the launchers that ran (name -> launches); classes nothing ran for are left out.
        Launchers no rule names are listed under "unclassified"."""
        rules = rules or DEFAULT_RULES
        out: Dict[str, Dict[str, int]] = {}
        seen = set()
        for cls, names in rules.items():
            hit = {n: self.counts[n] for n in names if n in self.counts}
            seen.update(hit)
            if hit:
                out[cls] = hit
        rest = {n: c for n, c in self.counts.items() if n not in seen}
        if rest:
            out["unclassified"] = rest
        return out

    def require(self, launcher: str, never: Iterable[str] = ()) -> None:
        """Raise unless ``launcher`` ran and none of ``never`` did."""
        if launcher not in self.counts:
            raise AssertionError(f"{launcher} never ran; ran: {sorted(self.counts)}")
        bad = [n for n in never if n in self.counts]
        if bad:
            raise AssertionError(f"{bad} ran although {launcher} should have served the op")
