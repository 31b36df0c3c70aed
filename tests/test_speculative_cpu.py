"""Speculative-decoding policies (pure host logic): draft-width ladder, capacity tiers, the
decode / verify throughput gate, adaptive rungs, D-Cut pruning, n-gram proposer. Mirrors the
reference's unit tests for ``crates/speculative`` and ``model-layers/src/speculative``."""
import pytest

from metrale_inference_alpha_b200.speculative.gate import MtpGate, SpecStats
from metrale_inference_alpha_b200.speculative.ladder import (AdaptiveRung, DflashRung, KLadder, dcut_plan,
                                                              spec_capacity, step_drafts)
from metrale_inference_alpha_b200.speculative.ngram import NgramProposer


def test_k_ladder_default_and_custom(monkeypatch):
    monkeypatch.delenv("METRALE_MTP_K_LADDER", raising=False)
    lad = KLadder()
    assert [lad.drafts_for(w) for w in (1, 4, 5, 8, 9, 16, 17, 32, 33, 128)] == [3, 3, 3, 3, 1, 1, 1, 1, 0, 0]
    assert KLadder("2:4,64:2", max_k=3).drafts_for(1) == 3
    assert KLadder("2:4,64:2").drafts_for(40) == 2
    monkeypatch.setenv("METRALE_MTP_K_LADDER", "128:2")
    assert KLadder().drafts_for(100) == 2


def test_capacity_tiers_bound_the_step_width():
    assert spec_capacity(0) == 3 and spec_capacity(7) == 3 and spec_capacity(8) == 1
    lad = KLadder("4:3,8:3,16:1,32:1")
    assert step_drafts([0, 1, 2], lad) == 3
    assert step_drafts([0, 1, 9], lad) == 1            # one narrow slot narrows the whole step
    assert step_drafts([], lad) == 0


def test_gate_measures_both_modes_then_settles_on_the_faster():
    g = MtpGate(window=4, dwell=1, margin=0.05)
    assert g.next_step() == MtpGate.MEASURE_VERIFY
    rate = {MtpGate.MEASURE_VERIFY: 100.0, MtpGate.MEASURE_DECODE: 150.0}
    seen = []
    for _ in range(80):
        m = g.next_step()
        seen.append(m)
        g.record(int(rate[m]), 1.0)
    assert MtpGate.MEASURE_DECODE in seen and seen[-1] == MtpGate.MEASURE_DECODE
    assert g.switches >= 1
    # and the other way round
    g = MtpGate(window=4, dwell=1)
    rate = {MtpGate.MEASURE_VERIFY: 220.0, MtpGate.MEASURE_DECODE: 150.0}
    for _ in range(80):
        g.record(int(rate[g.next_step()]), 1.0)
    assert g.next_step() == MtpGate.MEASURE_VERIFY


def test_gate_hysteresis_ignores_small_differences_and_disabled_gate_is_decode():
    g = MtpGate(window=2, dwell=1, margin=0.10)
    rate = {MtpGate.MEASURE_VERIFY: 100.0, MtpGate.MEASURE_DECODE: 104.0}
    for _ in range(12):
        g.record(int(rate[g.next_step()]), 1.0)
    s0 = g.switches
    for _ in range(40):
        g.record(int(rate[g.next_step()]), 1.0)
    assert g.switches == s0                              # 4 % is inside the margin: no flapping
    off = MtpGate(enabled=False)
    off.record(10, 1.0)
    assert off.next_step() == MtpGate.MEASURE_DECODE


def test_spec_stats_rates():
    s = SpecStats()
    s.steps, s.emitted, s.drafted, s.accepted = 10, 25, 30, 15
    assert s.accept_len == pytest.approx(2.5) and s.accept_rate == pytest.approx(0.5)


def test_adaptive_rung_enters_and_leaves_with_hysteresis():
    r = AdaptiveRung()
    assert r.drafts(4) == 1 and r.drafts(20) == 1
    for _ in range(80):
        r.observe(True, True)
    assert r.drafts(12) == 2
    for _ in range(80):
        r.observe(True, False)
    assert r.drafts(12) == 1


def test_dflash_rung_width():
    d = DflashRung()
    assert d.gamma(4) == d.multi
    assert d.gamma(1) == d.narrow
    for _ in range(64):
        d.observe(True)
    assert d.gamma(1) == d.wide
    for _ in range(64):
        d.observe(False)
    assert d.gamma(1) == d.narrow


def test_dcut_keeps_first_draft_and_cuts_suffix_closed():
    lps = [[-0.1, -0.2, -3.0], [-0.05, -0.05, -0.05], [-2.0, -2.5, -0.1]]
    assert dcut_plan(lps, 1.0) == [3, 3, 3]
    half = dcut_plan(lps, 0.5)
    assert all(k >= 1 for k in half) and sum(half) < 9
    assert half[1] == 3                                  # the confident sequence keeps its drafts
    assert half[2] == 1                                  # the unsure one is cut back to the first draft
    q = dcut_plan(lps, 0.25)
    assert sum(q) <= sum(half)
    # verify-row cap is enforced even at ratio 1
    wide = [[-0.1, -0.2, -0.3]] * 100
    plan = dcut_plan(wide, 1.0, row_cap=256)
    assert sum(plan) + len(plan) <= 256 and min(plan) >= 1


def test_ngram_proposer_prefers_longest_most_recent_match():
    p = NgramProposer(max_n=3, min_n=2)
    toks = [1, 2, 3, 9, 9, 1, 2, 3, 7, 8, 5, 1, 2, 3]
    assert p.propose(toks, 2) == [7, 8]
    assert p.propose(toks, 0) == []
    assert p.propose([1, 2], 3) == []
    assert p.propose([4, 5, 6, 7], 3) == []
