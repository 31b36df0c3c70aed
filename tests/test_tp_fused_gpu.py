"""Consumer-fused tensor-parallel reduction (ops/csrc/tp_fused.cu) on ONE GPU.

The ranks of a group are emulated inside one kernel launch: the kernel sums `emulate` local
partial buffers through the same peer-load path it uses across NVLink, and the barrier counts
this rank's own signals, so nothing waits on another launch. Checked against the fp32
reference: bf16(sum of partials) + residual -> RMSNorm -> encoder, and the pair merge of the
vocabulary-sharded argmax. The last test makes a bounded wait run out on a counter nobody
signals and checks that the status word reports it while the context stays usable."""
import pytest
import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.ops import reference as ref
from metrale_inference_alpha_b200.parallel.fused import FusedReduce, PendingSum

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _deq(a, M, K):
    if a.fmt == "bf16":
        return a.data.float().cpu()
    if a.fmt == "fp8_row":
        return ref.from_e4m3(a.data.cpu()) * a.scale.cpu()[:, None]
    if a.fmt == "fp8_g128":
        return ref.from_e4m3(a.data.cpu()) * a.scale.cpu()[:, :M].t().repeat_interleave(128, 1)[:, :K]
    nb = (M + 127) // 128
    sf = ref.tiled_to_sf(a.sf.cpu()[:nb * a.sf_k64 * 512].view(nb, a.sf_k64, 512), M, K // 16)
    return ref.dequantize_nvfp4(a.data.cpu(), sf, a.scale.cpu())


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8_row", "fp8_g128", "bf16"])
@pytest.mark.parametrize("ranks,M,K", [(1, 5, 1024), (4, 37, 5120), (8, 128, 2048), (2, 130, 7168)])
def test_reduce_norm_matches_reference(fmt, ranks, M, K):
    g = torch.Generator().manual_seed(11)
    fr = FusedReduce(0, 1, DEV, K, 160, emulate=ranks)
    w = (torch.randn(K, generator=g) * 0.1).to(torch.bfloat16)
    for it in range(3):                                   # consecutive calls alternate buffer parity
        parts = [(torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16) for _ in range(ranks)]
        res = torch.randn(M, K, generator=g).to(torch.bfloat16)
        for r, p in enumerate(parts):
            fr.partial_view(M, r).copy_(p.to(DEV))
        pend = PendingSum(fr, fr.partial_view(M, 0), res.to(DEV))
        a = fr.reduce_norm(pend, w.to(DEV), fmt, plus_one=True, eps=1e-6, also_bf16=True, gather_residual=True)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        s = ref.bf16_round(sum(p.float() for p in parts))
        h = ref.bf16_round(s + res.float())
        assert torch.equal(pend.value.cpu().float(), h), (pend.value.cpu().float() - h).abs().max()
        a_ref = ops.row_op(h.to(torch.bfloat16), fmt, ops.IN_RMSNORM, w=w, plus_one=True, eps=1e-6, also_bf16=True)[0]
        err = (a.bf16.float().cpu() - a_ref.bf16.float()).abs()
        assert (err <= 1e-2 + 1e-2 * a_ref.bf16.float().abs()).all()
        deq = _deq(a, M, K)
        step = a_ref.data.abs().amax(dim=1, keepdim=True) * (0.3 if fmt == "nvfp4" else 0.08)
        assert ((deq - a_ref.data).abs() <= step + 1e-3).all()
        assert ((deq - a_ref.data).abs() > 1e-3).float().mean() < 0.02
    fr.end_forward()


@pytest.mark.parametrize("M,K", [(1, 5120), (9, 2048), (64, 1024)])
def test_packet_protocol_loopback_matches_reference(M, K):
    """World size 1: the rank broadcasts its packets into its own landing zone and polls them
    back; repeated calls alternate the zone parity and change the tag."""
    g = torch.Generator().manual_seed(21)
    fr = FusedReduce(0, 1, DEV, K, 64)
    fr.force_proto = 2
    w = (torch.randn(K, generator=g) * 0.1).to(torch.bfloat16)
    for it in range(4):
        part = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
        res = torch.randn(M, K, generator=g).to(torch.bfloat16)
        fr.partial_view(M).copy_(part.to(DEV))
        pend = PendingSum(fr, fr.partial_view(M), res.to(DEV))
        a = fr.reduce_norm(pend, w.to(DEV), "nvfp4", eps=1e-6, also_bf16=True)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        h = ref.bf16_round(part.float() + res.float())
        assert torch.equal(pend.value.cpu().float(), h)
        a_ref = ops.row_op(h.to(torch.bfloat16), "nvfp4", ops.IN_RMSNORM, w=w, eps=1e-6, also_bf16=True)[0]
        deq = _deq(a, M, K)
        step = a_ref.data.abs().amax(dim=1, keepdim=True) * 0.3
        assert ((deq - a_ref.data).abs() <= step + 1e-3).all()
        assert ((deq - a_ref.data).abs() > 1e-3).float().mean() < 0.02


def test_reduce_without_norm_and_feeds_a_gemm():
    """resolve(): sum + residual only; and the NVFP4 rows the kernel wrote are a valid GEMM operand."""
    g = torch.Generator().manual_seed(5)
    M, K, N = 16, 2048, 512
    fr = FusedReduce(0, 1, DEV, K, 64, emulate=3)
    parts = [(torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16) for _ in range(3)]
    res = torch.randn(M, K, generator=g).to(torch.bfloat16)
    for r, p in enumerate(parts):
        fr.partial_view(M, r).copy_(p.to(DEV))
    pend = PendingSum(fr, fr.partial_view(M, 0), res.to(DEV))
    full = pend.resolve()
    h = ref.bf16_round(ref.bf16_round(sum(p.float() for p in parts)) + res.float())
    assert torch.equal(full.cpu().float(), h)
    for r, p in enumerate(parts):
        fr.partial_view(M, r).copy_(p.to(DEV))
    pend = PendingSum(fr, fr.partial_view(M, 0), res.to(DEV))
    wn = (torch.randn(K, generator=g) * 0.1).to(torch.bfloat16)
    a = fr.reduce_norm(pend, wn.to(DEV), "nvfp4", eps=1e-6)
    wq = ops.make_weight(torch.randn(N, K, generator=g) * 0.05, "nvfp4")
    got = ops.linear(a, wq.to(DEV), out_f32=True).cpu()
    want = _deq(a, M, K) @ wq.dequant().t()
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert (got - want).abs().max() <= 1e-2 * want.abs().max() + 1e-3


def test_argmax_merge_single_rank_matches_argmax():
    g = torch.Generator().manual_seed(9)
    M, V = 33, 18992
    fr = FusedReduce(0, 1, DEV, 1024, 64)
    lg = torch.randn(M, V, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.zeros(M, dtype=torch.int32, device=DEV)
    feed = torch.zeros(M, dtype=torch.int32, device=DEV)
    fr.argmax_merge(lg, 1000, out, feed)
    torch.cuda.synchronize()
    want = ops.argmax(lg).cpu() + 1000
    assert torch.equal(out.cpu(), want) and torch.equal(feed.cpu(), want)
    ops.check_status(DEV)


def test_bounded_wait_expires_and_reports():
    """A barrier whose second rank never signals: the wait runs out after its run-time cycle
    budget (about 1 ms here), the status word reads MB_ST_TIMEOUT_PEER, the data phase is
    skipped, and the next kernel on the same context runs normally."""
    fr = FusedReduce(0, 1, DEV, 1024, 16, emulate=2, wait_cycles=2_000_000)
    dummy = torch.zeros(64, dtype=torch.int32, device=DEV)
    real_sync = fr._sync

    def one_sided(status_ptr):
        s = real_sync(status_ptr)
        s.arrive_peer[1] = dummy.data_ptr()            # the "peer's" signal goes nowhere this rank looks
        return s
    fr._sync = one_sided
    rt = ops.runtime(DEV)
    rt.status.zero_()
    fr.partial_view(4, 0).fill_(1.0)
    fr.partial_view(4, 1).fill_(1.0)
    pend = PendingSum(fr, fr.partial_view(4, 0), None)
    fr.reduce_norm(pend, None, "none", do_norm=False, gather_residual=True)
    torch.cuda.synchronize()
    assert int(rt.status[0].item()) == 0x400
    with pytest.raises(Exception, match="device status"):
        ops.check_status(DEV)                           # raises and clears
    x = torch.randn(8, 1024, device=DEV).to(torch.bfloat16)
    y = ops.row_op(x, "bf16", ops.IN_COPY)[0].data
    torch.cuda.synchronize()
    assert torch.equal(x, y)
    assert ops.check_status(DEV) == 0
