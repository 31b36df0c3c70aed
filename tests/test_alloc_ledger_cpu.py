"""Allocation ledger and red zones."""
import gc

import pytest
import torch

from metrale_inference_alpha_b200.utils import alloc_ledger as AL


def test_ledger_records_sizes_sites_and_forgets_dead_tensors():
    led = AL.AllocLedger(0)
    a = led.alloc((4, 8), torch.float32, "cpu", "pool a")
    b = led.alloc(100, torch.uint8, "cpu", "pool b")
    c = led.alloc(28, torch.uint8, "cpu", "pool b")
    led.track(torch.zeros(10), "foreign")
    keep = led.report()
    assert keep[0] == {"name": "pool a", "site": keep[0]["site"], "device": "cpu", "count": 1, "bytes": 128}
    assert keep[1]["name"] == "pool b" and keep[1]["count"] == 2 and keep[1]["bytes"] == 128
    assert "test_alloc_ledger_cpu.py" in keep[0]["site"] and led.total_bytes() == 128 + 128          # `foreign` died at once
    assert float(a.sum()) == 0 and led.slack("cpu") is None
    del b, c
    gc.collect()
    assert [r["name"] for r in led.report()] == ["pool a"]


def test_red_zone_names_the_overrun_buffer():
    led = AL.AllocLedger(64)
    a = led.alloc((3, 5), torch.float32, "cpu", "victim")              # 60 bytes: padded to 64 before the band
    b = led.alloc(32, torch.uint8, "cpu", "bystander")
    assert led.check() == [] and float(a.sum()) == 0 and a.shape == (3, 5)
    # a write past the end of `victim`, through its own storage
    raw = torch.empty(0, dtype=torch.uint8).set_(a.untyped_storage())
    raw[64 + 3] = 7
    raw[64 + 10] = 9
    bad = led.check()
    assert len(bad) == 1 and bad[0]["name"] == "victim" and bad[0]["bytes_overwritten"] == 2 and bad[0]["first_offset"] == 3
    led.refill()
    assert led.check() == [] and int(b.sum()) == 0
    with pytest.raises(ValueError):
        AL.AllocLedger(10)


def test_engine_pools_are_in_the_ledger_and_a_damaged_band_latches_the_fault(monkeypatch):
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    led = AL.reset_for_tests(256)
    try:
        monkeypatch.setenv("METRALE_REDZONE_EVERY", "2")
        eng = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device="cpu", num_kv_blocks=32, max_num_seqs=2))
        rep = eng.memory_report()
        names = {r["name"] for r in rep["allocations"]}
        assert {"kv pool (k)", "kv pool (v)", "state pool (ssm)", "state pool (conv)"} <= names and rep["redzone_bytes"] == 256
        out = eng.generate([[5, 6, 7, 8, 9]], SamplingParams(max_tokens=5, temperature=0.0))
        assert len(out[0].output_ids) == 5 and eng.check_red_zones() == [] and not eng.fault.is_set()
        k0 = eng.runner.kv.k[0]
        raw = torch.empty(0, dtype=torch.uint8).set_(k0.untyped_storage())
        raw[k0.numel() * k0.element_size() + 5] = 1                 # one byte past the pool
        bad = eng.check_red_zones()
        assert bad and bad[0]["name"] == "kv pool (k)" and eng.fault.is_set() and "kv pool (k)" in eng.fault.reason()
    finally:
        AL.reset_for_tests(0)


def test_kernel_audit_counts_and_classifies_launchers():
    from metrale_inference_alpha_b200.ops import _native
    from metrale_inference_alpha_b200.utils.kernel_audit import KernelAudit
    with KernelAudit() as a:
        _native.check(0, "gemm[nvfp4 M=1 N=8 K=8]")
        _native.check(0, "gemm[bf16 M=2 N=8 K=8]")
        _native.check(0, "attn_prefill_tc")
        _native.check(0, "brand_new_kernel")
        with pytest.raises(_native.KernelError):
            _native.check(-1, "row_op")                      # a refused launch is not counted
    assert a.counts == {"gemm": 2, "attn_prefill_tc": 1, "brand_new_kernel": 1}
    res = a.resolve()
    assert res["gemm"] == {"gemm": 2} and res["prefill attention"] == {"attn_prefill_tc": 1} and res["unclassified"] == {"brand_new_kernel": 1}
    a.require("attn_prefill_tc", never=["paged_attention"])
    with pytest.raises(AssertionError):
        a.require("paged_attention")
    _native.check(0, "gemm")                                  # outside the audit: not counted
    assert a.counts["gemm"] == 2


def test_a_finalizer_that_runs_inside_a_locked_section_does_not_deadlock():
    """Garbage collection can run a dead tensor's finalizer on the thread that is inside the ledger's lock."""
    import threading

    from metrale_inference_alpha_b200.utils.alloc_ledger import AllocLedger
    led = AllocLedger()
    t = led.alloc((4,), torch.float32, "cpu", name="a")
    done = []

    def inside():
        with led._lock:                       # what alloc() holds when the collector fires
            led._drop(0)                      # the finalizer's body
        done.append(1)
    th = threading.Thread(target=inside, daemon=True)
    th.start()
    th.join(5)
    assert done, "the finalizer blocked on the ledger's own lock"
    del t
    assert led.total_bytes() == 0
