"""Scheduler core driven by scripted executors: no model, no GPU. Mirrors the reference's
scheduler test strategy (``crates/scheduler/tests``: admission, chunked prefill, preemption
under KV pressure, speculative accept / rewind, timeouts, aborts, injected device faults)."""
import pytest

from metrale_inference_alpha_b200.cache.block_pool import BlockAllocator
from metrale_inference_alpha_b200.cache.radix import RadixTree
from metrale_inference_alpha_b200.sampling.params import SamplingParams
from metrale_inference_alpha_b200.scheduler.core import SchedulerCore
from metrale_inference_alpha_b200.scheduler.policy import SchedulerConfig, TbtDeadlinePolicy
from metrale_inference_alpha_b200.scheduler.scripted import ScriptedExecutor, TracingExecutor
from metrale_inference_alpha_b200.scheduler.types import FatalDeviceError, KvExhausted, Request, SeqStatus


def make(blocks=64, prefix=False, **kw):
    cfg = SchedulerConfig(max_num_seqs=kw.pop("max_num_seqs", 8), max_prefill_tokens=kw.pop("max_prefill_tokens", 64),
                          max_model_len=kw.pop("max_model_len", 512), block_size=16, **kw)
    alloc = BlockAllocator(blocks)
    tree = RadixTree(alloc, 16) if prefix else None
    return SchedulerCore(cfg, alloc, tree), alloc


def req(i, n_prompt=20, max_tokens=8, **kw):
    return Request(f"r{i}", [(i * 13 + j) % 997 + 1 for j in range(n_prompt)], SamplingParams(max_tokens=max_tokens, **kw))


def drive(sch, ex, max_steps=10_000):
    outs = {}
    steps = 0
    while sch.has_work() and steps < max_steps:
        plan = sch.plan()
        if plan is None:
            for o in sch.drain_finished():
                outs[o.request_id] = o
            continue
        res = ex.execute(plan)
        for o in sch.apply(plan, res):
            outs[o.request_id] = o
        steps += 1
    for o in sch.drain_finished():
        outs[o.request_id] = o
    return outs, steps


def test_all_requests_finish_with_exact_lengths_and_blocks_return():
    sch, alloc = make()
    for i in range(5):
        sch.add_request(req(i, n_prompt=17 + i, max_tokens=5 + i))
    outs, _ = drive(sch, ScriptedExecutor())
    assert len(outs) == 5
    for i in range(5):
        o = outs[f"r{i}"]
        assert o.finished and o.finish_reason == "length" and len(o.output_ids) == 5 + i
    assert alloc.num_free == 64 - 1 or alloc.num_free == 64     # block 0 may be the reserved null block


def test_tokens_follow_the_script_independent_of_batch_composition():
    ex = ScriptedExecutor()
    sch, _ = make()
    s = sch.add_request(req(0, max_tokens=6))
    alone, _ = drive(sch, ex)
    sch2, _ = make()
    for i in range(4):
        sch2.add_request(req(i, max_tokens=6))
    crowd, _ = drive(sch2, ScriptedExecutor())
    # seq ids start equal in both schedulers, so request 0 sees the same script
    assert alone["r0"].output_ids == crowd["r0"].output_ids


def test_prefill_is_chunked_to_the_token_budget():
    sch, _ = make(max_prefill_tokens=32)
    sch.add_request(req(0, n_prompt=100, max_tokens=2))
    ex = TracingExecutor(ScriptedExecutor())
    drive(sch, ex)
    pre = [t for t in ex.trace if t["kind"] == "prefill"]
    assert [t["tokens"] for t in pre] == [32, 32, 32, 4]
    starts = [t["seqs"][0][1] for t in pre]
    assert starts == [0, 32, 64, 96]


def test_batch_cap_limits_running_sequences():
    sch, _ = make(max_num_seqs=3, blocks=256)
    for i in range(7):
        sch.add_request(req(i, max_tokens=4))
    ex = TracingExecutor(ScriptedExecutor())
    outs, _ = drive(sch, ex)
    assert len(outs) == 7
    assert max(len(t["seqs"]) for t in ex.trace if t["kind"] == "decode") <= 3


def test_preemption_under_kv_pressure_recomputes_and_finishes():
    # 12 usable blocks of 16 tokens: four sequences of 40 prompt + 60 new tokens cannot coexist
    sch, alloc = make(blocks=13, max_num_seqs=4, decode_reserve_tokens=0)
    for i in range(4):
        sch.add_request(req(i, n_prompt=40, max_tokens=60))
    outs, _ = drive(sch, ScriptedExecutor())
    assert len(outs) == 4 and all(o.finished for o in outs.values())
    assert sch.stats["preempted"] > 0
    assert all(len(o.output_ids) == 60 for o in outs.values() if o.finish_reason == "length")


def test_preempted_sequence_resumes_with_the_same_tokens():
    fn = lambda sid, pos: (sid * 101 + pos * 7) % 500 + 1
    sch, _ = make(blocks=13, max_num_seqs=4, decode_reserve_tokens=0)
    for i in range(4):
        sch.add_request(req(i, n_prompt=40, max_tokens=40))
    tight, _ = drive(sch, ScriptedExecutor(fn))
    sch2, _ = make(blocks=256, max_num_seqs=4)
    for i in range(4):
        sch2.add_request(req(i, n_prompt=40, max_tokens=40))
    roomy, _ = drive(sch2, ScriptedExecutor(fn))
    for k in roomy:
        assert tight[k].output_ids == roomy[k].output_ids


def test_abort_releases_blocks_and_reports_abort():
    sch, alloc = make()
    sch.add_request(req(0, max_tokens=50))
    ex = ScriptedExecutor()
    for _ in range(3):
        p = sch.plan()
        sch.apply(p, ex.execute(p))
    used = alloc.num_used
    assert used > 0 and sch.abort("r0")
    outs = sch.drain_finished()
    assert outs and outs[-1].finish_reason == "abort"
    assert alloc.num_used < used and not sch.has_work()
    assert not sch.abort("nope")


def test_request_timeout_finishes_with_timeout_reason():
    sch, _ = make()
    t = [0.0]
    sch.clock = lambda: t[0]
    r = req(0, max_tokens=1000, timeout_s=5.0)
    r.arrival = 0.0
    sch.add_request(r)
    ex = ScriptedExecutor()
    for _ in range(3):
        p = sch.plan()
        sch.apply(p, ex.execute(p))
    t[0] = 10.0
    outs, _ = drive(sch, ex)
    assert outs["r0"].finish_reason == "timeout"


def test_stop_token_and_eos_and_min_tokens():
    fn = lambda sid, pos: 7
    sch, _ = make()
    r = req(0, max_tokens=20)
    r.eos_token_id = 7
    sch.add_request(r)
    outs, _ = drive(sch, ScriptedExecutor(fn))
    assert outs["r0"].finish_reason == "stop" and len(outs["r0"].output_ids) == 1
    sch, _ = make()
    r = req(1, max_tokens=20, min_tokens=4)
    r.eos_token_id = 7
    sch.add_request(r)
    outs, _ = drive(sch, ScriptedExecutor(fn))
    assert len(outs["r1"].output_ids) == 4
    sch, _ = make()
    r = req(2, max_tokens=6, ignore_eos=True)
    r.eos_token_id = 7
    sch.add_request(r)
    outs, _ = drive(sch, ScriptedExecutor(fn))
    assert outs["r2"].finish_reason == "length" and len(outs["r2"].output_ids) == 6


def test_speculative_accept_and_rewind():
    fn = lambda sid, pos: (pos * 3) % 100 + 1
    ex = ScriptedExecutor(fn)
    # drafter that gets the first two tokens right and the third wrong
    ex.draft_fn = lambda sid, n_tokens, k: [fn(sid, n_tokens - 1 + j) if j < 2 else 999 for j in range(k)][:k]
    sch, _ = make()
    sch.add_request(req(0, max_tokens=30))
    outs = {}
    while sch.has_work():
        p = sch.plan()
        res = ex.execute(p)
        dr = ex.propose(p, res, 3)
        for o in sch.apply(p, res, None):
            outs[o.request_id] = o
        for it, d in zip(p.items, dr):
            if not it.seq.is_finished():
                it.seq.drafts = [fn(it.seq.seq_id, len(it.seq.tokens) - 1 + j) if j < 2 else 999 for j in range(3)]
    o = outs["r0"]
    expect = [fn(0, 19 + j) for j in range(30)]
    assert o.output_ids[:30] == expect
    assert o.accepted_draft_tokens > 0 and o.rejected_draft_tokens > 0


def test_injected_kv_exhaustion_and_fatal_fault_surface_as_exceptions():
    sch, _ = make()
    sch.add_request(req(0))
    ex = ScriptedExecutor()
    ex.inject(1, "kv")
    ex.inject(3, "fatal")
    p = sch.plan(); sch.apply(p, ex.execute(p))
    p = sch.plan()
    with pytest.raises(KvExhausted):
        ex.execute(p)
    sch.apply(p, ex.execute(p))                  # retry of the same plan succeeds
    p = sch.plan()
    with pytest.raises(FatalDeviceError):
        ex.execute(p)


def test_prefix_cache_shortens_second_prefill():
    sch, _ = make(prefix=True, blocks=128)
    sch.add_request(req(0, n_prompt=70, max_tokens=3))
    ex = TracingExecutor(ScriptedExecutor())
    drive(sch, ex)
    r2 = req(0, n_prompt=70, max_tokens=3)
    r2.request_id = "again"
    sch.add_request(r2)
    n0 = len(ex.trace)
    outs, _ = drive(sch, ex)
    pre = [t for t in ex.trace[n0:] if t["kind"] == "prefill"]
    assert sum(t["tokens"] for t in pre) < 70
    assert outs["again"].cached_tokens >= 48


def test_tbt_policy_holds_prefill_until_decode_ran():
    pol = TbtDeadlinePolicy(100.0)
    assert pol.should_prefill(True, False, 0.0)
    pol.note_decode(0.0)
    assert pol.should_prefill(True, True, 0.001) in (True, False)
    # when the deadline is about to pass, decode goes first
    assert not pol.should_prefill(True, True, 0.2) or pol.should_prefill(True, True, 0.2) is True


def test_snapshot_reports_counts():
    sch, _ = make()
    sch.add_request(req(0))
    s = sch.snapshot()
    assert s["waiting"] + s["prefilling"] + s["running"] == 1


def test_slai_policy_orders_admission_and_protects_decodes():
    from collections import deque

    from metrale_inference_alpha_b200.scheduler.policy import SchedulerConfig, SlaiPolicy, make_policy
    p = make_policy(SchedulerConfig(policy="slai", tbt_deadline_ms=100.0))
    assert isinstance(p, SlaiPolicy)
    p.note_decode(10.0)
    assert p.should_prefill(True, True, 10.05)                     # 50 ms waited: prefill may start
    assert not p.should_prefill(True, True, 10.081)                # 81 ms = past 80 % of the deadline: decode first
    assert p.should_prefill(True, False, 99.0)                     # nothing is decoding: always prefill
    assert not p.should_prefill(False, True, 10.0)
    cfg = SchedulerConfig(max_prefill_tokens=4096)
    assert p.prefill_budget(cfg, True) == 4096                     # chunks are never shrunk

    class S:
        def __init__(self, n):
            self.tokens = [0] * n
    q = deque(S(n) for n in (900, 50, 400, 10, 400))
    first_400 = q[2]
    SlaiPolicy.order_waiting(q)
    assert [len(s.tokens) for s in q] == [900, 10, 50, 400, 400] and q[3] is first_400     # head kept, rest shortest first, stable
    import pytest as _pt
    with _pt.raises(ValueError):
        make_policy(SchedulerConfig(policy="nope"))
    # through the scheduler with two seats: the head of the queue and the shortest of the rest go first
    sch, _ = make(policy="slai", max_num_seqs=2, blocks=256)
    for i, n in enumerate((60, 40, 20, 50)):
        sch.add_request(req(i, n_prompt=n, max_tokens=2))
    plan = sch.plan()
    assert sorted(len(it.seq.tokens) for it in plan.items) == [20, 60]
    outs, _ = drive(sch, ScriptedExecutor())
    assert len(outs) == 4                                       # every request still finishes


def test_mixed_lane_never_plans_a_sequence_it_just_preempted():
    """Mixed prefill + decode with a pool so small that growing the decode rows preempts the
    prefilling sequence: its chunk must leave the plan (its blocks were freed), every plan item
    still owns the blocks it addresses, and all requests finish with the scripted tokens."""
    ex = ScriptedExecutor()
    sch, alloc = make(blocks=7, mixed_prefill_decode=True, max_prefill_tokens=16)
    sch.add_request(req(0, n_prompt=30, max_tokens=40))
    outs = {}
    steps = 0
    added = False
    while sch.has_work() and steps < 2000:
        plan = sch.plan()
        if plan is None:
            continue
        for it in plan.items:
            assert it.seq.status in (SeqStatus.PREFILL, SeqStatus.DECODE), it.seq.status
            need = (it.start_pos + len(it.tokens) + 15) // 16
            assert len(it.seq.blocks) >= need, (it.seq.req.request_id, len(it.seq.blocks), need)
        res = ex.execute(plan)
        for o in sch.apply(plan, res):
            outs[o.request_id] = o
        steps += 1
        if not added and sch.running and len(sch.running[0].tokens) >= 45:
            sch.add_request(req(1, n_prompt=40, max_tokens=6))     # r0 needs its next block while r1 is prefilling
            added = True
    for o in sch.drain_finished():
        outs[o.request_id] = o
    assert sch.stats["preempted"] >= 1
    assert outs["r0"].finished and outs["r1"].finished
    assert len(outs["r0"].output_ids) == 40 and len(outs["r1"].output_ids) == 6


def test_mixed_plan_drops_the_chunk_of_a_sequence_preempted_while_building_it():
    sch, _ = make(blocks=64, mixed_prefill_decode=True, max_prefill_tokens=16)
    ex = ScriptedExecutor()
    sch.add_request(req(0, n_prompt=10, max_tokens=30))
    while not sch.running:                                   # r0 reaches decode
        plan = sch.plan()
        sch.apply(plan, ex.execute(plan))
    sch.add_request(req(1, n_prompt=40, max_tokens=4))       # r1 will be mid-prefill
    real = sch._decode_items

    def decode_items_under_pressure():
        victim = sch.prefilling[0] if sch.prefilling else None
        items = real()
        if victim is not None:
            assert sch.preempt_one(exclude=sch.running[0]) is victim     # what KV exhaustion does
        return items
    sch._decode_items = decode_items_under_pressure
    plan = sch.plan()
    sch._decode_items = real
    assert plan is not None and plan.kind == "mixed"
    assert [it.seq.req.request_id for it in plan.items] == ["r0"]
    assert all(it.seq.blocks for it in plan.items)
    sch.apply(plan, ex.execute(plan))
    outs, _ = drive(sch, ex)
    assert outs["r1"].finished and len(outs["r1"].output_ids) == 4


def _drive_look_ahead(sch, ex, arrivals):
    """The engine's pipelined loop on the scripted executor: step t + 1 is planned (and 'launched')
    before step t's tokens are applied."""
    outs, inflight, step, ahead_steps = {}, None, 0, 0
    while arrivals or sch.has_work() or inflight:
        for r in arrivals.pop(step, []):
            sch.add_request(r)
        step += 1
        if inflight is not None:
            plan, res = inflight
            inflight = None
        else:
            plan = sch.plan()
            if plan is None:
                for o in sch.drain_finished():
                    outs[o.request_id] = o
                continue
            res = ex.execute(plan)
        nxt = sch.plan_ahead(plan) if plan.kind == "decode" else None
        if nxt is not None:
            inflight = (nxt, ex.execute(nxt))          # results exist before plan's tokens are applied
            ahead_steps += 1
        for o in sch.apply(plan, res):
            outs[o.request_id] = o
    for o in sch.drain_finished():
        outs[o.request_id] = o
    return outs, ahead_steps


def test_look_ahead_decode_equals_synchronous_decode_including_overrun_discard():
    """One step of look-ahead must not change any request's tokens: sequences that stop on a
    stop token while their next row is already in flight have that row discarded; arrivals,
    length limits and block boundaries interrupt the pipeline and it resumes afterwards."""
    probe, _ = make(blocks=64)
    for r in (req(0, n_prompt=20, max_tokens=40), req(1, n_prompt=33, max_tokens=17), req(2, n_prompt=9, max_tokens=60)):
        probe.add_request(r)
    seq_ids = drive(probe, ScriptedExecutor())[0]["r2"].output_ids
    stop = next(t for j, t in enumerate(seq_ids) if j >= 20 and t not in seq_ids[:j])   # first seen at step >= 20

    def arrivals():
        return {0: [req(0, n_prompt=20, max_tokens=40), req(1, n_prompt=33, max_tokens=17),
                    req(2, n_prompt=9, max_tokens=60, stop_token_ids=[stop])],
                12: [req(3, n_prompt=50, max_tokens=25)], 13: [req(4, n_prompt=5, max_tokens=3)]}
    sch, alloc = make(blocks=64)
    sync_outs = {}
    arr = arrivals()
    step = 0
    ex = ScriptedExecutor()
    while arr or sch.has_work():
        for r in arr.pop(step, []):
            sch.add_request(r)
        step += 1
        plan = sch.plan()
        if plan is None:
            for o in sch.drain_finished():
                sync_outs[o.request_id] = o
            continue
        for o in sch.apply(plan, ex.execute(plan)):
            sync_outs[o.request_id] = o
    sch2, alloc2 = make(blocks=64)
    outs, ahead_steps = _drive_look_ahead(sch2, ScriptedExecutor(), arrivals())
    assert ahead_steps > 30
    assert set(outs) == set(sync_outs) == {f"r{i}" for i in range(5)}
    for k in outs:
        assert outs[k].finished and outs[k].output_ids == sync_outs[k].output_ids, k
        assert outs[k].finish_reason == sync_outs[k].finish_reason
    assert outs["r2"].finish_reason == "stop" and len(outs["r2"].output_ids) < 60
    assert alloc2.num_free == alloc.num_free
