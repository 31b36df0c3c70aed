"""Recurrent-state and MoE kernels against their fp32 PyTorch references."""
import pytest
import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.config.model_config import preset
from metrale_inference_alpha_b200.engine.batch import ForwardBatch
from metrale_inference_alpha_b200.ops import moe as moe_ops
from metrale_inference_alpha_b200.ops import recurrent as rops
from metrale_inference_alpha_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, rtol=2e-3, atol=2e-3):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    assert (err <= atol + rtol * want.abs()).all(), f"max err {err.max():.4g} (ref max {want.abs().max():.4g})"


def _batch(dev):
    # three sequences: fresh prefill (7 tokens), continuing decode (1 token at position 5), verify (3 at pos 9)
    seqs = [dict(tokens=[1] * 7, start_pos=0, blocks=[1], state_slot=1),
            dict(tokens=[2], start_pos=5, blocks=[2], state_slot=2),
            dict(tokens=[3] * 3, start_pos=9, blocks=[3], state_slot=3)]
    return ForwardBatch.build(seqs, 16, device=dev)


def test_causal_conv1d_matches_reference():
    g = torch.Generator().manual_seed(0)
    C, taps, T = 200, 4, 11
    x = torch.randn(T, C + 24, generator=g).to(torch.bfloat16)
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g)
    st = torch.randn(5, C, taps - 1, generator=g)
    st_ref = st.clone()
    want = rops.causal_conv1d(x, C, w, b, st_ref, _batch("cpu"))
    st_dev = st.to(DEV)
    got = rops.causal_conv1d(x.to(DEV), C, w.to(DEV), b.to(DEV), st_dev, _batch(DEV))
    _close(got, want)
    _close(st_dev, st_ref)


@pytest.mark.parametrize("taps", [2, 4])
def test_time_parallel_conv1d_matches_the_sequential_reference(taps):
    """Prefill chunks (>= 64 tokens) take the time-parallel kernel + the state kernel: outputs and the
    stored window must equal the CPU reference for fresh sequences, continuations from a stored
    window, sequences shorter than the window and a one-token sequence in the same launch."""
    g = torch.Generator().manual_seed(3)
    C = 200
    lens = [200, 1, 77, 64, 2]
    seqs = [dict(tokens=[1] * n, start_pos=0 if i % 2 == 0 else 9, blocks=list(range(1, 3 + n // 16)), state_slot=i + 1)
            for i, n in enumerate(lens)]
    T = sum(lens)
    x = torch.randn(T, C + 24, generator=g).to(torch.bfloat16)
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    st = torch.randn(len(lens) + 1, C, taps - 1, generator=g)
    st_ref = st.clone()
    want = rops.causal_conv1d(x, C, w, b, st_ref, ForwardBatch.build(seqs, 16, device="cpu"))
    st_dev = st.to(DEV)
    n0 = ops.launch_count
    got = rops.causal_conv1d(x.to(DEV), C, w.to(DEV), b.to(DEV), st_dev, ForwardBatch.build(seqs, 16, device=DEV))
    assert ops.launch_count - n0 == 2                       # the parallel kernel and the state kernel
    _close(got, want)
    _close(st_dev, st_ref)
    assert torch.equal(st_dev[0].cpu(), st[0])              # untouched slot


@pytest.mark.parametrize("dk", [32, 128])
def test_gdn_recurrence_matches_reference(dk):
    g = torch.Generator().manual_seed(1)
    kh, vh, T = 2, 4, 11
    QK, V = kh * dk, vh * dk
    conv = torch.randn(T, 2 * QK + V, generator=g)
    ba = torch.randn(T, 2 * vh, generator=g)
    A_log, dtb = torch.randn(vh, generator=g) * 0.3, torch.randn(vh, generator=g) * 0.1
    st = torch.randn(5, vh, dk, dk, generator=g) * 0.1
    st_ref = st.clone()
    want = rops.gdn_recurrence(conv, ba, A_log, dtb, st_ref, _batch("cpu"), k_heads=kh, v_heads=vh, k_dim=dk, v_dim=dk)
    st_dev = st.to(DEV)
    got = rops.gdn_recurrence(conv.to(DEV), ba.to(DEV), A_log.to(DEV), dtb.to(DEV), st_dev, _batch(DEV),
                              k_heads=kh, v_heads=vh, k_dim=dk, v_dim=dk)
    _close(got, want, 5e-3, 5e-3)
    _close(st_dev, st_ref, 5e-3, 5e-3)


@pytest.mark.parametrize("N,P", [(16, 32), (128, 64)])
def test_mamba2_scan_matches_reference(N, P):
    g = torch.Generator().manual_seed(2)
    H, G, T = 8, 2, 11
    inner, GN = H * P, G * N
    xbc = torch.randn(T, inner + 2 * GN, generator=g)
    dt = torch.randn(T, H + 8, generator=g).to(torch.bfloat16)
    A_log, D, dtb = torch.randn(H, generator=g) * 0.3, torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.1
    st = torch.randn(5, H, P, N, generator=g) * 0.1
    st_ref = st.clone()
    kw = dict(heads=H, groups=G, head_dim=P, state=N)
    want = rops.mamba2_scan(xbc, dt[:, :H], A_log, D, dtb, st_ref, _batch("cpu"), **kw)
    st_dev = st.to(DEV)
    got = rops.mamba2_scan(xbc.to(DEV), dt.to(DEV)[:, :H], A_log.to(DEV), D.to(DEV), dtb.to(DEV), st_dev,
                           _batch(DEV), **kw)
    _close(got, want, 5e-3, 5e-3)
    _close(st_dev, st_ref, 5e-3, 5e-3)


@pytest.mark.parametrize("lens", [[64], [200, 1, 77], [8192], [130, 64, 5, 300]])
def test_mamba2_chunked_scan_matches_the_sequential_kernel_and_the_fp32_oracle(lens):
    """State-space-dual chunked scan (TF32 tensor-core products) against the sequential kernel on
    the same inputs: outputs and the hand-off state; the shortest case also against the fp32 CPU
    reference. Sequences mix fresh starts with continuations from a stored state."""
    g = torch.Generator().manual_seed(12)
    H, G, P, N = 16, 2, 64, 128
    inner, GN = H * P, G * N
    seqs, pos = [], 0
    for i, n in enumerate(lens):
        seqs.append(dict(tokens=[1] * n, start_pos=0 if i % 2 == 0 else 7, blocks=list(range(1, 2 + (n + 7) // 16)), state_slot=i + 1))
    b = ForwardBatch.build(seqs, 16, device=DEV)
    T = sum(lens)
    xbc = (torch.randn(T, inner + 2 * GN, generator=g) * 0.5).to(DEV)
    dt = (torch.randn(T, H + 8, generator=g) * 0.5).to(torch.bfloat16).to(DEV)[:, :H]
    A_log = (torch.randn(H, generator=g) * 0.3).to(DEV)
    Dv, dtb = torch.randn(H, generator=g).to(DEV), (torch.randn(H, generator=g) * 0.1).to(DEV)
    s0 = (torch.randn(len(lens) + 1, H, P, N, generator=g) * 0.1).to(DEV)
    kw = dict(heads=H, groups=G, head_dim=P, state=N)
    st_seq, st_chk = s0.clone(), s0.clone()
    rops._SSD_MIN_TOKENS, keep = 1 << 30, rops._SSD_MIN_TOKENS
    want = rops.mamba2_scan(xbc, dt, A_log, Dv, dtb, st_seq, b, **kw)          # sequential kernel
    rops._SSD_MIN_TOKENS = 1
    got = rops.mamba2_scan(xbc, dt, A_log, Dv, dtb, st_chk, b, **kw)           # chunked kernels
    rops._SSD_MIN_TOKENS = keep
    torch.cuda.synchronize()
    ops.check_status(DEV)
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 4e-3 * max(1.0, scale), ((got - want).abs().max().item(), scale)
    assert (st_chk - st_seq).abs().max().item() <= 4e-3 * max(1.0, st_seq.abs().max().item())
    assert torch.equal(st_chk[0], s0[0])                                       # untouched slot
    if T <= 64:
        st_cpu = s0.cpu().clone()
        ref_y = rops.mamba2_scan(xbc.cpu(), dt.cpu(), A_log.cpu(), Dv.cpu(), dtb.cpu(), st_cpu,
                                 ForwardBatch.build(seqs, 16, device="cpu"), **kw)
        _close(got, ref_y, 5e-3, 5e-3 * max(1.0, scale))
        _close(st_chk, st_cpu, 5e-3, 5e-3)


@pytest.mark.parametrize("lens", [[64], [200, 1, 77], [8192], [130, 64, 5, 300]])
def test_gdn_chunked_prefill_matches_the_sequential_kernel_and_the_fp32_oracle(lens):
    """Chunked gated delta rule (WY form, TF32 tensor-core products) against the sequential kernel
    on the same inputs: outputs and the hand-off state; the shortest case also against the fp32
    CPU reference. Sequences mix fresh starts with continuations from a stored state, and the
    decay / beta gates cover both strong forgetting and near-1 retention."""
    g = torch.Generator().manual_seed(14)
    kh, vh, dk = 2, 4, 128
    QK, V = kh * dk, vh * dk
    seqs = []
    for i, n in enumerate(lens):
        seqs.append(dict(tokens=[1] * n, start_pos=0 if i % 2 == 0 else 7, blocks=list(range(1, 2 + (n + 7) // 16)), state_slot=i + 1))
    b = ForwardBatch.build(seqs, 16, device=DEV)
    T = sum(lens)
    conv = torch.randn(T, 2 * QK + V, generator=g).to(DEV)
    ba = (torch.randn(T, 2 * vh, generator=g) * 1.5).to(DEV)
    A_log = (torch.randn(vh, generator=g) * 0.5).to(DEV)
    dtb = (torch.randn(vh, generator=g) * 0.3).to(DEV)
    s0 = (torch.randn(len(lens) + 1, vh, dk, dk, generator=g) * 0.1).to(DEV)
    kw = dict(k_heads=kh, v_heads=vh, k_dim=dk, v_dim=dk)
    st_seq, st_chk = s0.clone(), s0.clone()
    rops._GDN_CHUNK_MIN_TOKENS, keep = 1 << 30, rops._GDN_CHUNK_MIN_TOKENS
    want = rops.gdn_recurrence(conv, ba, A_log, dtb, st_seq, b, **kw)           # sequential kernel
    rops._GDN_CHUNK_MIN_TOKENS = 1
    n0 = ops.launch_count
    got = rops.gdn_recurrence(conv, ba, A_log, dtb, st_chk, b, **kw)            # chunked kernels
    assert ops.launch_count - n0 == 2
    rops._GDN_CHUNK_MIN_TOKENS = keep
    torch.cuda.synchronize()
    ops.check_status(DEV)
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 5e-3 * max(1.0, scale), ((got - want).abs().max().item(), scale)
    assert (st_chk - st_seq).abs().max().item() <= 5e-3 * max(1.0, st_seq.abs().max().item())
    assert torch.equal(st_chk[0], s0[0])                                       # untouched slot
    if T <= 64:
        st_cpu = s0.cpu().clone()
        ref_y = rops.gdn_recurrence(conv.cpu(), ba.cpu(), A_log.cpu(), dtb.cpu(), st_cpu,
                                    ForwardBatch.build(seqs, 16, device="cpu"), **kw)
        _close(got, ref_y, 5e-3, 5e-3 * max(1.0, scale))
        _close(st_chk, st_cpu, 5e-3, 5e-3)


def _commit_batch(b, n_rows):
    import dataclasses
    return dataclasses.replace(b, q_len=torch.tensor(n_rows, dtype=torch.int32, device=b.q_len.device))


@pytest.mark.parametrize("dev", ["cpu", DEV])
def test_write_on_accept_equals_feeding_only_the_accepted_rows(dev):
    """Speculative verify over the recurrent kernels: a pass with write_state=False leaves the
    state untouched and gives the same outputs; the commit pass (q_len = accepted rows,
    write_out=False) leaves exactly the state that feeding only those rows would have left,
    bit for bit (same kernel, same order of operations)."""
    g = torch.Generator().manual_seed(4)
    b = _batch(dev)                                     # q_len 7 (fresh), 1, 3
    accept = [4, 1, 0]                                  # rows committed per sequence (0: nothing accepted yet)
    T = 11
    # conv
    C, taps = 200, 4
    x = torch.randn(T, C, generator=g).to(torch.bfloat16).to(dev)
    w, bias = torch.randn(C, taps, generator=g).to(dev), torch.randn(C, generator=g).to(dev)
    st0 = torch.randn(5, C, taps - 1, generator=g).to(dev)
    full_state = st0.clone()
    full = rops.causal_conv1d(x, C, w, bias, full_state, b)
    st = st0.clone()
    ver = rops.causal_conv1d(x, C, w, bias, st, b, write_state=False)
    assert torch.equal(st, st0) and torch.equal(ver, full)
    rops.causal_conv1d(x, C, w, bias, st, _commit_batch(b, accept), write_out=False)
    want = st0.clone()
    rops.causal_conv1d(x, C, w, bias, want, _commit_batch(b, accept))
    assert torch.equal(st, want)
    assert torch.equal(st[3], st0[3]) and not torch.equal(st[1], st0[1])
    # gated delta net
    kh, vh, dk = 2, 4, 32
    QK, V = kh * dk, vh * dk
    conv = torch.randn(T, 2 * QK + V, generator=g).to(dev)
    ba = torch.randn(T, 2 * vh, generator=g).to(dev)
    A_log, dtb = (torch.randn(vh, generator=g) * 0.3).to(dev), (torch.randn(vh, generator=g) * 0.1).to(dev)
    s0 = (torch.randn(5, vh, dk, dk, generator=g) * 0.1).to(dev)
    kw = dict(k_heads=kh, v_heads=vh, k_dim=dk, v_dim=dk)
    fs = s0.clone()
    full = rops.gdn_recurrence(conv, ba, A_log, dtb, fs, b, **kw)
    st = s0.clone()
    ver = rops.gdn_recurrence(conv, ba, A_log, dtb, st, b, write_state=False, **kw)
    assert torch.equal(st, s0) and torch.equal(ver, full)
    rops.gdn_recurrence(conv, ba, A_log, dtb, st, _commit_batch(b, accept), write_out=False, **kw)
    want = s0.clone()
    rops.gdn_recurrence(conv, ba, A_log, dtb, want, _commit_batch(b, accept), **kw)
    assert torch.equal(st, want) and torch.equal(st[3], s0[3])
    # Mamba2
    H, G, P, N = 8, 2, 32, 16
    inner, GN = H * P, G * N
    xbc = torch.randn(T, inner + 2 * GN, generator=g).to(dev)
    dt = torch.randn(T, H + 8, generator=g).to(torch.bfloat16).to(dev)[:, :H]
    A_log, D, dtb = (torch.randn(H, generator=g) * 0.3).to(dev), torch.randn(H, generator=g).to(dev), (torch.randn(H, generator=g) * 0.1).to(dev)
    s0 = (torch.randn(5, H, P, N, generator=g) * 0.1).to(dev)
    kw = dict(heads=H, groups=G, head_dim=P, state=N)
    fs = s0.clone()
    full = rops.mamba2_scan(xbc, dt, A_log, D, dtb, fs, b, **kw)
    st = s0.clone()
    ver = rops.mamba2_scan(xbc, dt, A_log, D, dtb, st, b, write_state=False, **kw)
    assert torch.equal(st, s0) and torch.equal(ver, full)
    rops.mamba2_scan(xbc, dt, A_log, D, dtb, st, _commit_batch(b, accept), write_out=False, **kw)
    want = s0.clone()
    rops.mamba2_scan(xbc, dt, A_log, D, dtb, want, _commit_batch(b, accept), **kw)
    assert torch.equal(st, want) and torch.equal(st[3], s0[3])
    if dev != "cpu":
        torch.cuda.synchronize()
        ops.check_status(DEV)


def test_router_softmax_and_group_limited():
    g = torch.Generator().manual_seed(3)
    T, E = 37, 256
    logits = torch.randn(T, E, generator=g)
    cfg = preset("qwen-hybrid-moe-35b-fp8")
    w_ref, i_ref = moe_ops.route(logits, cfg)
    w, i = moe_ops.route(logits.to(DEV), cfg)
    assert torch.equal(i.cpu(), i_ref)
    _close(w, w_ref, 1e-4, 1e-6)
    cfg = preset("deepseek-v3-671b-fp8")
    bias = torch.randn(E, generator=g) * 0.1
    w_ref, i_ref = moe_ops.route(logits, cfg, bias)
    w, i = moe_ops.route(logits.to(DEV), cfg, bias.to(DEV))
    assert torch.equal(i.cpu().sort(-1).values, i_ref.sort(-1).values)
    _close(w.cpu().sort(-1).values, w_ref.sort(-1).values, 1e-4, 1e-6)


@pytest.mark.parametrize("fmt", ["fp8_block", "fp8_row", "bf16"])
def test_grouped_expert_ffn_matches_loop(fmt):
    from metrale_inference_alpha_b200.models.decoder import Decoder
    from metrale_inference_alpha_b200.models.moe import routed_experts
    from metrale_inference_alpha_b200.weights.loader import FfnW, MoeW
    g = torch.Generator().manual_seed(4)
    T, H, I, E, K = 29, 256, 128, 8, 2
    cfg = preset("qwen-hybrid-moe-35b-fp8", num_layers=1, hidden_size=H, num_experts=E, experts_per_token=K,
                 moe_intermediate_size=I, weight_format=fmt, vocab_size=512)
    experts = []
    for e in range(E):
        gate, up = torch.randn(I, H, generator=g) * 0.05, torch.randn(I, H, generator=g) * 0.05
        down = torch.randn(H, I, generator=g) * 0.05
        if fmt == "fp8_block":
            gu, inter = ops.make_weight(torch.cat([gate, up]), fmt), False
        else:
            gu, inter = ops.make_weight(ops.interleave_gate_up(gate, up), fmt), True
        experts.append(FfnW(gu, ops.make_weight(down, fmt), interleaved=inter))
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, K, generator=g)

    class _D:
        pass
    d = _D(); d.cfg = cfg
    a_ref = ops.quantize_act(x, ops.ACT_FOR_WEIGHT[fmt])
    want = routed_experts(d, a_ref, wts, idx, MoeW(experts=experts))
    dev_experts = [FfnW(e.gate_up.to(DEV), e.down.to(DEV), e.interleaved) for e in experts]
    mw = MoeW(experts=dev_experts, grouped=moe_ops.stack_experts(dev_experts))
    a = ops.quantize_act(x.to(DEV), ops.ACT_FOR_WEIGHT[fmt])
    got = routed_experts(d, a, wts.to(DEV), idx.to(DEV), mw)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    _close(got, want, 3e-2, 3e-2 * want.abs().max().item())


# ---------------------------------------------------------------------------- absorbed MLA attention
@pytest.mark.parametrize("impl", [1, 2])
@pytest.mark.parametrize("H,q_lens,ctx_lens,part_tokens", [
    (16, [1, 1, 1], [5, 130, 64], 0),             # decode, ragged contexts, one row group per sequence
    (128, [1, 1], [700, 33], 0),                  # DeepSeek-V3 head count: 8 row groups
    (8, [4, 1, 7], [40, 9, 200], 0),              # verify / chunked rows: causal limits inside a group
    (16, [1, 2], [300, 257], 128),                # three partitions + merge kernel
    (128, [1, 1, 1], [1000, 31, 257], 256),       # decode with partitions (the tcgen05 kernel + merge)
    (40, [1], [97], 0),                           # a head count that does not fill the 128-row tile
])
def test_mla_attention_matches_fp32_oracle(H, q_lens, ctx_lens, part_tokens, impl):
    """impl 1 = the mma.sync kernel, 2 = the tcgen05 / TMEM decode kernel (one query row per sequence,
    16 <= H <= 128; other cases are skipped for it)."""
    if impl == 2 and (max(q_lens) != 1 or H < 16):
        pytest.skip("the tcgen05 kernel serves decode rows")
    from types import SimpleNamespace
    from metrale_inference_alpha_b200.models.mla import mla_attention as mla_ref
    from metrale_inference_alpha_b200.ops import mla_cuda
    g = torch.Generator().manual_seed(11)
    bs, D, L = 16, 576, 512
    S = len(q_lens)
    nblk = [(c + bs - 1) // bs for c in ctx_lens]
    nb = sum(nblk) + 1
    cache = (torch.randn(nb, bs, 1, D, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.zeros(S, max(nblk) + 2, dtype=torch.int32)
    perm = (torch.randperm(nb - 1, generator=g) + 1).tolist()
    k = 0
    for s in range(S):
        for b in range(nblk[s]):
            bt[s, b] = perm[k]
            k += 1
    T = sum(q_lens)
    q = (torch.randn(T, H, D, generator=g) * 0.5).to(torch.bfloat16)
    qs = torch.tensor([sum(q_lens[:i]) for i in range(S)], dtype=torch.int32)
    ql, cl = torch.tensor(q_lens, dtype=torch.int32), torch.tensor(ctx_lens, dtype=torch.int32)
    batch = SimpleNamespace(q_start=qs, q_len=ql, ctx_len=cl, block_table=bt)
    scale = 1.0 / (192 ** 0.5)
    want = mla_ref(q, cache, batch, scale, L)
    got = mla_cuda.mla_attention(q.to(DEV), cache.to(DEV), bt.to(DEV), qs.to(DEV), ql.to(DEV), cl.to(DEV),
                                 max_q_len=max(q_lens), max_ctx=max(ctx_lens), scale=scale, part_tokens=part_tokens,
                                 impl=impl)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    err = (got.cpu() - want).abs().max().item()
    assert err < 2e-2 * max(1.0, want.abs().max().item()), err


# ---------------------------------------------------------------------------- LoRA shrink / expand
def test_lora_kernels_match_cpu_manager():
    from metrale_inference_alpha_b200.lora import LoraAdapter, LoraManager
    g = torch.Generator().manual_seed(4)
    dims = {"o": (1024, 520), "k": (1024, 256)}
    cpu = LoraManager(2, dims, max_adapters=4, max_rank=16)
    gpu = LoraManager(2, dims, max_adapters=4, max_rank=16, device=DEV)
    for i, r in enumerate((8, 16, 4)):
        w = {(l, t): ((torch.randn(r, dims[t][0], generator=g) * 0.1).bfloat16(),
                      (torch.randn(dims[t][1], r, generator=g) * 0.1).bfloat16()) for l in range(2) for t in dims}
        for m in (cpu, gpu):
            m.load(LoraAdapter(f"a{i}", r, alpha=2.0 * r, weights=w))
    M = 37
    x = torch.randn(M, 1024, generator=g).bfloat16()
    rows = torch.tensor([(-1, 0, 1, 2)[i % 4] for i in range(64)], dtype=torch.int32)
    for layer, target, col0, width in ((0, "o", 0, 520), (1, "k", 128, 640)):
        base = torch.randn(M, width, generator=g).bfloat16()
        want = base.clone()
        cpu.apply(want, x.float(), layer, target, rows, col0)
        got = base.to(DEV)
        gpu.apply(got, x.to(DEV), layer, target, rows.to(DEV), col0)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        assert torch.allclose(got.float().cpu(), want.float(), rtol=2e-2, atol=2e-2)
        untouched = [m for m in range(M) if rows[m] < 0]
        assert torch.equal(got.cpu()[untouched], base[untouched])


def test_engine_with_adapters_on_gpu_isolates_rows():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.lora import LoraAdapter
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    cfg = preset("tiny-dense")
    D = cfg.head_dim

    def tensors(seed, zero_b):
        g = torch.Generator().manual_seed(seed)
        t = {}
        for l in range(cfg.num_layers):
            for tg, (K, N) in {"q": (cfg.hidden_size, cfg.num_heads * D), "v": (cfg.hidden_size, cfg.num_kv_heads * D),
                               "o": (cfg.num_heads * D, cfg.hidden_size), "down": (cfg.intermediate_size, cfg.hidden_size)}.items():
                grp = "mlp" if tg == "down" else "self_attn"
                t[f"base_model.model.model.layers.{l}.{grp}.{tg}_proj.lora_A.weight"] = torch.randn(4, K, generator=g) * 0.5
                t[f"base_model.model.model.layers.{l}.{grp}.{tg}_proj.lora_B.weight"] = (
                    torch.zeros(N, 4) if zero_b else torch.randn(N, 4, generator=g) * 0.5)
        return t
    eng = LLMEngine(EngineArgs(model=cfg, device=DEV, max_num_seqs=4, max_model_len=128))
    eng.load_adapter("noop", LoraAdapter.from_tensors("noop", tensors(1, True), 4, 8.0))
    eng.load_adapter("strong", LoraAdapter.from_tensors("strong", tensors(2, False), 4, 8.0))
    prompt, sp = [3, 4, 5, 6, 7, 8, 9, 10], SamplingParams(max_tokens=6)

    def run(adapters):
        ids = [eng.add_request(prompt, sp, adapter=a) for a in adapters]
        res = {}
        while eng.has_work():
            for o in eng.step():
                if o.finished:
                    res[o.request_id] = o.output_ids
        return [res[i] for i in ids]
    base = run([None])[0]                          # CUDA-graph decode path
    assert run(["noop"])[0] == base                # eager path with a zero delta: same tokens
    mixed = run([None, "strong", "noop"])
    assert mixed[0] == base and mixed[2] == base and mixed[1] != base
    assert run(["strong"])[0] == mixed[1]          # the adapted row does not depend on its neighbours
    ops.check_status(DEV)


# ---------------------------------------------------------------------------- EP all-to-all (one rank = loopback)
def test_ep_all_to_all_loopback_matches_local_experts():
    """World size 1: the dispatch / return kernels run against the rank's own landing zone, so the
    whole protocol (slots, counts, flags, parity double buffering) is exercised on one GPU and the
    result must equal the local routed-expert path."""
    from metrale_inference_alpha_b200.parallel.ep import EpAllToAll
    torch.manual_seed(0)
    T, K, H, E = 23, 2, 256, 8
    x = torch.randn(T, H, device=DEV).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=DEV)[:K] for _ in range(T)]).to(torch.int32)
    wts = torch.rand(T, K, device=DEV)
    mats = torch.randn(E, H, H, device=DEV) * 0.05

    def expert_fn(rows, eids):
        e = eids.view(-1).long()
        out = torch.zeros(rows.shape[0], H, device=DEV)
        ok = e >= 0
        out[ok] = torch.einsum("nh,nhk->nk", rows[ok].float(), mats[e[ok]])
        return out
    ep = EpAllToAll(0, 1, DEV, hidden=H, max_tokens=32, top_k=K)
    want = torch.zeros(T, H, device=DEV)
    for j in range(K):
        want += wts[:, j:j + 1] * torch.einsum("nh,nhk->nk", x.float(), mats[idx[:, j].long()])
    for step in range(3):                                  # alternating parities, stale zones from earlier steps
        got = ep.moe(x, wts, idx, E, expert_fn)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        assert torch.allclose(got, want, rtol=3e-2, atol=3e-2 * want.abs().max().item()), step
        x = x.flip(0).contiguous()
        idx = idx.flip(0).contiguous()
        wts = wts.flip(0).contiguous()
        want = want.flip(0)


def test_mla_block_on_gpu_matches_the_cpu_restatement():
    """A two-layer DeepSeek-shaped model with the real latent geometry (512 + 64) through the
    engine on both devices: the GPU block (bf16 absorption products, the operand-assembly kernel,
    the paged MLA kernel) must give the logits of the fp32 restatement on CPU, for a prefill
    and for decode steps over the cache rows the assembly kernel wrote."""
    from metrale_inference_alpha_b200.config.model_config import from_hf_config
    from metrale_inference_alpha_b200.engine.runner import ModelRunner
    from metrale_inference_alpha_b200.scheduler.policy import SchedulerConfig
    from metrale_inference_alpha_b200.weights.loader import load_weights
    cfg = from_hf_config(dict(model_type="deepseek_v3", vocab_size=1024, hidden_size=512, num_hidden_layers=2,
                              num_attention_heads=16, num_key_value_heads=16, intermediate_size=512, moe_intermediate_size=128,
                              n_routed_experts=0, first_k_dense_replace=2, kv_lora_rank=512, q_lora_rank=192,
                              qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, rms_norm_eps=1e-6, rope_theta=1e4,
                              max_position_embeddings=512), name="tiny-mla")
    toks = torch.randint(1, 1024, (37,), generator=torch.Generator().manual_seed(8)).tolist()
    logits = {}
    from metrale_inference_alpha_b200.weights.source import SyntheticSource
    for dev in ("cpu", DEV):
        w = load_weights(cfg, SyntheticSource(cfg, seed=3, device="cpu"), device=dev)      # the same checkpoint on both devices
        r = ModelRunner(cfg, w, dev, num_blocks=16, sched=SchedulerConfig(max_num_seqs=2, max_model_len=256), use_graphs=False)
        blocks = [1, 2, 3, 4]
        out = []
        b = ForwardBatch.build([dict(tokens=toks, start_pos=0, blocks=blocks, state_slot=0)], 16, device=dev, max_blocks=r.max_blocks)
        lg, _ = r.decoder.forward(b, r.caches, out_f32=True)
        out.append(lg.float().cpu())
        nxt = int(lg.argmax())
        for step in range(3):                                   # decode rows read what the prefill wrote
            b = ForwardBatch.build([dict(tokens=[nxt], start_pos=len(toks) + step, blocks=blocks, state_slot=0)], 16,
                                   device=dev, max_blocks=r.max_blocks)
            lg, _ = r.decoder.forward(b, r.caches, out_f32=True)
            out.append(lg.float().cpu())
            nxt = int(out[0].argmax()) if step < 0 else 7 + step   # fixed tokens: both devices see the same inputs
        logits[dev] = out
    if DEV == "cuda":
        torch.cuda.synchronize()
        ops.check_status(DEV)
    for a, bb in zip(logits["cpu"], logits[DEV]):
        assert (a - bb).abs().max() <= 0.04 * a.abs().max() + 2e-3, ((a - bb).abs().max(), a.abs().max())
        assert int(a.argmax()) == int(bb.argmax())


# ----------------------------------------------------------------------------- storage tier kernels
@pytest.mark.parametrize("D,fp8", [(128, False), (128, True), (256, False), (256, True)])
def test_kv_tile_attention_folds_tiles_like_the_restatement(D, fp8):
    from metrale_inference_alpha_b200.storage import kernels as SK
    g = torch.Generator().manual_seed(3)
    S, Hq, Hkv, bs, nblk = 3, 8, 2, 16, 12
    k = torch.randn(nblk, bs, Hkv, D, generator=g) * 0.5
    v = torch.randn(nblk, bs, Hkv, D, generator=g)
    if fp8:
        pk, pv = k.to(torch.float8_e4m3fn).view(torch.uint8), v.to(torch.float8_e4m3fn).view(torch.uint8)
        ks, vs = 0.5, 2.0
    else:
        pk, pv, ks, vs = k.to(torch.bfloat16), v.to(torch.bfloat16), 1.0, 1.0
    q = torch.randn(S, Hq, D, generator=g).to(torch.bfloat16)
    tiles = [(torch.tensor([[0, 5, 2, 7], [1, 3, 0, 0], [4, 6, 8, 9]], dtype=torch.int32), torch.tensor([4, 2, 4], dtype=torch.int32),
              torch.tensor([16, 9, 16], dtype=torch.int32)),
             (torch.tensor([[10, 11, 0, 0], [0, 0, 0, 0], [3, 0, 0, 0]], dtype=torch.int32), torch.tensor([2, 0, 1], dtype=torch.int32),
              torch.tensor([3, 16, 1], dtype=torch.int32))]
    strides = SK.paged_strides(bs, Hkv, D)
    outs = {}
    for dev in ("cpu", DEV):
        st = SK.attn_state(S, Hq, D, dev)
        fused = torch.zeros(S, Hq, D, dtype=torch.bfloat16, device=dev)
        for i, (tb, tc, lv) in enumerate(tiles):
            SK.kv_tile_attn(q.to(dev), pk.to(dev), pv.to(dev), tb.to(dev), tc.to(dev), st, Hkv=Hkv, block_size=bs,
                            strides=strides, last_valid=lv.to(dev), k_scale=ks, v_scale=vs,
                            out=fused if i == len(tiles) - 1 else None)
        outs[dev] = (SK.attn_finalize(st[1], st[2]), fused, st)
    _close(outs[DEV][0], outs["cpu"][0], 2e-2, 2e-2)
    _close(outs[DEV][1], outs["cpu"][0], 2e-2, 2e-2)            # the last tile's fused output = finalize
    _close(outs[DEV][2][0], outs["cpu"][2][0], 1e-3, 1e-3)      # running maxima


def test_lowrank_projection_and_predictor_score_match_the_restatement():
    from metrale_inference_alpha_b200.storage import kernels as SK
    g = torch.Generator().manual_seed(4)
    Hq, Hkv, D, bs, r, nblk = 8, 2, 128, 16, 32, 10
    P = (torch.randn(D, r, generator=g) / D ** 0.5).to(torch.bfloat16)
    q = torch.randn(3, Hq, D, generator=g).to(torch.bfloat16)
    _close(SK.project_rows(q.to(DEV), P.to(DEV)), SK.project_rows(q, P), 2e-2, 2e-2)
    for fp8 in (False, True):
        k = torch.randn(nblk, bs, Hkv, D, generator=g)
        pool = k.to(torch.float8_e4m3fn).view(torch.uint8) if fp8 else k.to(torch.bfloat16)
        src = torch.tensor([7, 2, 9], dtype=torch.int32)
        dst = torch.tensor([1, 4, 0], dtype=torch.int32)
        lr = {}
        for dev in ("cpu", DEV):
            out = torch.zeros(6, Hkv, bs, r, dtype=torch.bfloat16, device=dev)
            SK.project_blocks(pool.to(dev), P.to(dev), out, src.to(dev), dst.to(dev), Hkv=Hkv, block_size=bs,
                              strides=SK.paged_strides(bs, Hkv, D), k_scale=0.5 if fp8 else 1.0)
            lr[dev] = out
        _close(lr[DEV], lr["cpu"], 2e-2, 2e-2)
    k_lr = lr["cpu"]
    q_lr = SK.project_rows(q, P)
    blocks = torch.tensor([[1, 4, 0, 0], [0, 1, 4, 0], [4, 0, 0, 0]], dtype=torch.int32)
    counts = torch.tensor([2, 3, 1], dtype=torch.int32)
    last = torch.tensor([5, 16, 1], dtype=torch.int32)
    want = SK.predictor_score(q_lr, k_lr, blocks, counts, last)
    got = SK.predictor_score(q_lr.to(DEV), k_lr.to(DEV), blocks.to(DEV), counts.to(DEV), last.to(DEV)).cpu()
    assert torch.equal(torch.isinf(got), torch.isinf(want))
    fin = ~torch.isinf(want)
    _close(got[fin], want[fin], 1e-2, 1e-2)


def test_streamed_attention_through_files_on_the_device(tmp_path):
    import math
    from metrale_inference_alpha_b200.storage import HighSpeedSwap, HighSpeedSwapConfig, ModelDims
    g = torch.Generator().manual_seed(5)
    md = ModelDims(1, 8, 2, 128)
    hss = HighSpeedSwap(HighSpeedSwapConfig(dir=str(tmp_path / "kv"), block_size=16, max_blocks_per_layer=64,
                                            resident_blocks=12, tile_capacity=4, rank=32, max_seqs=2), md, device=DEV)
    lens, ids, kv = [200, 96], [], []
    for n in lens:
        k = (torch.randn(n, 2, 128, generator=g) * 0.5).to(torch.bfloat16)
        v = torch.randn(n, 2, 128, generator=g).to(torch.bfloat16)
        nb = (n + 15) // 16
        d = [hss.alloc_disk_block() for _ in range(nb)]
        for j, blk in enumerate(d):
            kb, vb = torch.zeros(16, 2, 128, dtype=torch.bfloat16), torch.zeros(16, 2, 128, dtype=torch.bfloat16)
            m = min(16, n - j * 16)
            kb[:m], vb[:m] = k[j * 16:j * 16 + m], v[j * 16:j * 16 + m]
            hss.offload_block(0, blk, kb.to(DEV), vb.to(DEV))
        ids.append(d)
        kv.append((k, v))
    q = torch.randn(2, 8, 128, generator=g).to(torch.bfloat16)
    last = [n - (len(d) - 1) * 16 for n, d in zip(lens, ids)]
    for _ in range(2):
        out = hss.attend_layer(0, q.to(DEV), ids, last_valid=last).float().cpu()
        for s, (k, v) in enumerate(kv):
            for h in range(8):
                sc = (k[:, h // 4].float() @ q[s, h].float()) / math.sqrt(128)
                ref_o = torch.softmax(sc, 0) @ v[:, h // 4].float()
                _close(out[s, h], ref_o, 2e-2, 2e-2)
    assert hss.stats["evictions"] > 0 and hss.stats["slot_hits"] > 0
    ops.check_status(torch.device(DEV))
    hss.close()


def test_paged_experts_grouped_path_matches_resident_experts(tmp_path, monkeypatch):
    """One MoE block on the device: experts paged through an arena smaller than the expert count (several
    waves per call, evictions between calls) against the same block with every expert resident."""
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.models.moe import moe_block
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.storage.expert_store import enable_expert_paging
    monkeypatch.setenv("METRALE_MOE_FOLD_SHARED", "0")          # the same block structure on both sides
    eng = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device=DEV, num_kv_blocks=64, max_num_seqs=4, use_cuda_graphs=False))
    dec = eng.runner.decoder
    lw = next(L for L in eng.weights.layers if L.ffn_kind == "moe")
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(n, eng.cfg.hidden_size, generator=g).to(torch.bfloat16).to(DEV) for n in (52, 3, 1)]
    want = [moe_block(dec, x, lw).float() for x in xs]
    paged = enable_expert_paging(eng.weights, str(tmp_path / "experts"), 3, DEV)
    got = [moe_block(dec, x, lw).float() for x in xs]
    for gy, wy in zip(got, want):
        _close(gy, wy, 2e-2, 2e-2)
    assert paged.stats["waves"] >= 4 and paged.stats["evictions"] > 0
    # and the engine serves with it
    out = eng.generate([list(range(5, 45))], SamplingParams(max_tokens=4, temperature=0.0))[0].output_ids
    assert len(out) == 4
    ops.check_status(torch.device(DEV))


# ----------------------------------------------------------------------------- Kimi delta attention
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("fused_norm", [False, True])
def test_kda_recurrence_matches_reference(D, fused_norm):
    g = torch.Generator().manual_seed(6)
    H, T = 3, 11
    conv = torch.randn(T, 3 * H * D, generator=g)
    g_raw = torch.randn(T, H * D, generator=g)
    b_raw = torch.randn(T, H, generator=g)
    A_log, dtb = torch.randn(H, generator=g) * 0.3, torch.randn(H * D, generator=g) * 0.3
    st = torch.randn(5, H, D, D, generator=g) * 0.1
    gate = torch.randn(T, H * D, generator=g).to(torch.bfloat16)
    w = torch.rand(D, generator=g) + 0.5
    outs = {}
    for dev in ("cpu", DEV):
        s = st.clone().to(dev)
        norm = (w.to(dev), gate.to(dev), 1e-6) if fused_norm else None
        y = rops.kda_recurrence(conv.to(dev), g_raw.to(dev), b_raw.to(dev), A_log.to(dev), dtb.to(dev), -5.0, s,
                                _batch(dev), heads=H, dim=D, norm=norm)
        outs[dev] = (y, s)
    tol = 2e-2 if fused_norm else 2e-3
    _close(outs[DEV][0], outs["cpu"][0], tol, tol)
    _close(outs[DEV][1], outs["cpu"][1], 2e-3, 2e-3)
    # a pass that writes no state leaves it untouched
    s2 = st.clone().to(DEV)
    rops.kda_recurrence(conv.to(DEV), g_raw.to(DEV), b_raw.to(DEV), A_log.to(DEV), dtb.to(DEV), -5.0, s2, _batch(DEV),
                        heads=H, dim=D, write_state=False)
    assert torch.equal(s2.cpu(), st)
    ops.check_status(torch.device(DEV))


def test_kimi_linear_model_runs_on_the_device_and_chunked_prefill_agrees():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    prompts = [list(range(5, 75)), list(range(40, 59))]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    whole = LLMEngine(EngineArgs(model="tiny-kimi-linear", device=DEV, num_kv_blocks=64, max_num_seqs=4))
    want = [o.output_ids for o in whole.generate(prompts, sp)]
    assert all(len(w) == 6 for w in want)
    graphs_off = LLMEngine(EngineArgs(model="tiny-kimi-linear", device=DEV, num_kv_blocks=64, max_num_seqs=4,
                                      use_cuda_graphs=False))
    assert [o.output_ids for o in graphs_off.generate(prompts, sp)] == want


# ----------------------------------------------------------------------------- sparse (indexed) attention
@pytest.mark.parametrize("Di,Hi", [(128, 64), (64, 4)])
def test_index_scores_match_the_restatement(Di, Hi):
    from metrale_inference_alpha_b200.ops import sparse_attn as SA
    g = torch.Generator().manual_seed(8)
    bs, nb = 16, 40
    kc = torch.randn(nb, bs, 1, Di, generator=g).to(torch.bfloat16)
    table = torch.randint(1, nb, (2, 24), generator=g, dtype=torch.int32)
    row_seq = torch.tensor([0, 0, 0, 1], dtype=torch.int32)
    row_ctx = torch.tensor([298, 299, 300, 77], dtype=torch.int32)
    iq = torch.randn(4, Hi, Di, generator=g).to(torch.bfloat16)
    iw = torch.rand(4, Hi, generator=g)
    want = SA.index_scores(iq, iw, kc, table, row_seq, row_ctx, 300)
    got = SA.index_scores(iq.to(DEV), iw.to(DEV), kc.to(DEV), table.to(DEV), row_seq.to(DEV), row_ctx.to(DEV), 300).cpu()
    assert got.shape == want.shape and torch.equal(torch.isinf(got), torch.isinf(want))
    fin = ~torch.isinf(want)
    _close(got[fin], want[fin], 2e-3, 2e-3)
    ops.check_status(torch.device(DEV))


def test_topk_selection_equals_a_stable_sort():
    from metrale_inference_alpha_b200.ops import sparse_attn as SA
    g = torch.Generator().manual_seed(9)
    T, n = 5, 5000
    sc = torch.randn(T, 5056, generator=g)
    sc[1] = torch.randint(0, 20, (5056,), generator=g).float()            # heavy ties
    sc[2, :] = 1.0                                                         # everything equal
    sc[3] = -sc[3].abs()                                                   # all negative
    ctx = torch.tensor([n, n, 4000, 3000, 37], dtype=torch.int32)
    for k in (64, 2048):
        want_i, want_c = SA.topk_indices(sc, ctx, k)
        got_i, got_c = SA.topk_indices(sc.to(DEV), ctx.to(DEV), k)
        assert torch.equal(got_c.cpu(), want_c)
        assert torch.equal(got_i.cpu(), want_i)


def test_selected_latent_attention_matches_the_restatement():
    from metrale_inference_alpha_b200.ops import sparse_attn as SA
    g = torch.Generator().manual_seed(10)
    bs, nb, H, W, L = 16, 64, 16, 576, 512
    cache = (torch.randn(nb, bs, 1, W, generator=g) * 0.3).to(torch.bfloat16)
    table = torch.randint(1, nb, (2, 40), generator=g, dtype=torch.int32)
    row_seq = torch.tensor([0, 1, 1], dtype=torch.int32)
    row_ctx = torch.tensor([600, 333, 334], dtype=torch.int32)
    sc = torch.randn(3, 640, generator=g)
    idx, cnt = SA.topk_indices(sc, row_ctx, 128)
    qq = (torch.randn(3, H, W, generator=g) * 0.3).to(torch.bfloat16)
    want = SA.selected_latent_attention(qq, cache, table, row_seq, idx, cnt, 0.05, L)
    got = SA.selected_latent_attention(qq.to(DEV), cache.to(DEV), table.to(DEV), row_seq.to(DEV), idx.to(DEV), cnt.to(DEV),
                                       0.05, L)
    _close(got, want, 2e-2, 2e-2)
    rows_d = SA.gather_rows(cache.to(DEV), table.to(DEV), row_seq.to(DEV), idx.to(DEV), cnt.to(DEV)).cpu()
    rows_h = SA.gather_rows(cache, table, row_seq, idx, cnt)
    n = int(cnt[0])
    assert torch.equal(rows_d.view(3, -1, W)[:, :n], rows_h.view(3, -1, W)[:, :n])
    ops.check_status(torch.device(DEV))


def test_sparse_mla_model_runs_on_the_device():
    import dataclasses
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    cfg = preset("deepseek-v3-671b-fp8", num_layers=3, first_dense_layers=1, hidden_size=512, num_heads=16,
                 num_kv_heads=16, q_lora_rank=256, dense_intermediate_size=1024, intermediate_size=1024,
                 num_experts=8, experts_per_token=2, moe_intermediate_size=256, router_n_group=2,
                 router_topk_group=1, vocab_size=4096, mtp_layers=0, max_position=1024,
                 index_topk=32, index_n_heads=4, index_head_dim=64)
    prompts = [list(range(5, 105)), list(range(200, 230))]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    eager = LLMEngine(EngineArgs(model=cfg, device=DEV, num_kv_blocks=64, max_num_seqs=4, use_cuda_graphs=False))
    want = [o.output_ids for o in eager.generate(prompts, sp)]
    graphs = LLMEngine(EngineArgs(model=cfg, device=DEV, num_kv_blocks=64, max_num_seqs=4))
    assert [o.output_ids for o in graphs.generate(prompts, sp)] == want
    # the selection covers the whole context: the dense kernel and the gather path see the same tokens
    wide = dataclasses.replace(cfg, index_topk=512)
    dense = LLMEngine(EngineArgs(model=wide, device=DEV, num_kv_blocks=64, max_num_seqs=4, use_cuda_graphs=False))
    assert all(len(o.output_ids) == 6 for o in dense.generate(prompts, sp))
    ops.check_status(torch.device(DEV))


# ----------------------------------------------------------------------------- residual highway
def test_hyper_connection_kernels_match_the_restatement():
    from metrale_inference_alpha_b200.ops import highway as hw
    g = torch.Generator().manual_seed(11)
    for hc, H, T in ((4, 1024, 7), (2, 512, 7), (4, 1024, 37), (4, 5120, 130)):           # few rows: one kernel; many: mix + finish
        streams = torch.randn(T, hc, H, generator=g)
        fn = (torch.randn((2 + hc) * hc, hc * H, generator=g) * 0.03).to(torch.bfloat16)
        scale, base = torch.tensor([1.0, 0.5, 2.0]), torch.randn((2 + hc) * hc, generator=g) * 0.1
        want = hw.hc_pre(streams, fn, scale, base, iters=6)
        got = hw.hc_pre(streams.to(DEV), fn.to(DEV), scale.to(DEV), base.to(DEV), iters=6)
        for a, b in zip(got, want):
            _close(a, b, 1e-2, 1e-2)
        out = torch.randn(T, H, generator=g).to(torch.bfloat16)
        s_d = hw.hc_post(out.to(DEV), streams.clone().to(DEV), want[1].to(DEV), want[2].to(DEV))
        _close(s_d, hw.hc_post(out, streams.clone(), want[1], want[2]), 1e-4, 1e-4)


def test_engram_ple_and_dilated_conv_kernels_match_the_restatement():
    from metrale_inference_alpha_b200.ops import highway as hw
    g = torch.Generator().manual_seed(12)
    T, hc, H = 11, 4, 512
    streams = torch.randn(T, hc, H, generator=g)
    kv = torch.randn(T, (hc + 1) * H, generator=g).to(torch.bfloat16)
    qk = torch.rand(hc, H, generator=g)
    _close(hw.engram_gate_add(streams.clone().to(DEV), kv.to(DEV), qk.to(DEV)), hw.engram_gate_add(streams.clone(), kv, qk),
           1e-3, 1e-3)
    key, value = torch.randn(T, hc * H, generator=g).to(torch.bfloat16), torch.randn(T, H, generator=g).to(torch.bfloat16)
    ws = [torch.randn(hc, H, generator=g) * 0.1 for _ in range(3)]
    want = hw.ple_gate(streams, key, value, *ws)
    got = hw.ple_gate(streams.to(DEV), key.to(DEV), value.to(DEV), *[w.to(DEV) for w in ws])
    _close(got[0], want[0], 1e-3, 1e-3)
    _close(got[1], want[1], 2e-3, 2e-3)
    C, taps, dil = hc * H, 4, 3
    w = torch.randn(C, taps, generator=g) * 0.3
    st = torch.randn(5, C, (taps - 1) * dil, generator=g)
    s_h, s_d = st.clone(), st.clone().to(DEV)
    o_h = hw.dilated_conv(want[1], want[0], w, s_h, _batch("cpu"), dil)
    o_d = hw.dilated_conv(want[1].to(DEV), want[0].to(DEV), w.to(DEV), s_d, _batch(DEV), dil)
    _close(o_d, o_h, 1e-3, 1e-3)
    _close(s_d, s_h, 1e-5, 1e-5)
    ops.check_status(torch.device(DEV))


def test_dense_model_on_a_highway_runs_on_the_device():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    prompts = [list(range(5, 60)), list(range(40, 52))]
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    eager = LLMEngine(EngineArgs(model="tiny-dense-hc", device=DEV, num_kv_blocks=64, max_num_seqs=4, use_cuda_graphs=False))
    want = [o.output_ids for o in eager.generate(prompts, sp)]
    graphs = LLMEngine(EngineArgs(model="tiny-dense-hc", device=DEV, num_kv_blocks=64, max_num_seqs=4))
    assert [o.output_ids for o in graphs.generate(prompts, sp)] == want


# ----------------------------------------------------------------------------- vision input
def test_vision_tower_on_the_device_matches_the_host_and_images_reach_the_model():
    import dataclasses
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.vision import VisionConfig, VisionEncoder
    vc = VisionConfig(depth=2, embed_dim=128, hidden_size=256, num_heads=4, mlp_ratio=2)
    t = VisionEncoder.random_tensors(vc, 3)
    g = torch.Generator().manual_seed(13)
    patches, grid = torch.randn(24 + 16, vc.patch_dim, generator=g), torch.tensor([[1, 4, 6], [2, 2, 4]])
    want = VisionEncoder(vc, t)(patches, grid)
    got = VisionEncoder(vc, t, device=DEV)(patches, grid)
    _close(got, want, 3e-2, 3e-2)
    cfg = dataclasses.replace(preset("tiny-dense"), image_token_id=4000, vision=dict(depth=1, embed_dim=64, num_heads=2, mlp_ratio=2),
                              name="tiny-vl")
    eng = LLMEngine(EngineArgs(model=cfg, device=DEV, num_kv_blocks=128, max_num_seqs=4, max_model_len=512))
    eng.attach_vision()
    img = torch.randint(0, 255, (56, 84, 3), generator=g, dtype=torch.uint8)
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    prompt = list(range(5, 19)) + [4000, 7, 8, 9]
    out = eng.generate([prompt, [5, 6, 7, 8]], sp, images=[[img], None])
    assert len(out[0].output_ids) == 6 and out[0].prompt_tokens == len(prompt) + 5
    again = eng.generate([prompt], sp, images=[[img]])[0]
    assert again.output_ids == out[0].output_ids and again.cached_tokens > 0
    ops.check_status(torch.device(DEV))


def test_nllb_on_the_device_matches_the_host():
    from metrale_inference_alpha_b200.models.nllb import NllbConfig, NllbModel
    g = torch.Generator().manual_seed(14)
    cfg = NllbConfig(vocab_size=512, d_model=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4,
                     decoder_attention_heads=4, encoder_ffn_dim=256, decoder_ffn_dim=256, max_position_embeddings=64)
    r = lambda *s: torch.randn(*s, generator=g) * 0.08
    t = {"shared.weight": r(512, 128)}
    for side, n in (("encoder", 2), ("decoder", 2)):
        for i in range(n):
            p = f"{side}.layers.{i}"
            atts = ["self_attn"] + (["encoder_attn"] if side == "decoder" else [])
            for a in atts:
                for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
                    t[f"{p}.{a}.{proj}.weight"], t[f"{p}.{a}.{proj}.bias"] = r(128, 128), r(128)
                t[f"{p}.{a}_layer_norm.weight"], t[f"{p}.{a}_layer_norm.bias"] = 1 + r(128), r(128)
            t[f"{p}.fc1.weight"], t[f"{p}.fc1.bias"], t[f"{p}.fc2.weight"], t[f"{p}.fc2.bias"] = r(256, 128), r(256), r(128, 256), r(128)
            t[f"{p}.final_layer_norm.weight"], t[f"{p}.final_layer_norm.bias"] = 1 + r(128), r(128)
        t[f"{side}.layer_norm.weight"], t[f"{side}.layer_norm.bias"] = 1 + r(128), r(128)
    host, dev = NllbModel(cfg, t), NllbModel(cfg, t, device=DEV)
    src = torch.tensor([[10, 11, 12, 13, 2], [10, 44, 2, 1, 1]])
    dec = torch.tensor([[2, 20, 31, 32], [2, 20, 41, 42]])
    want = host.decode_step(dec, host.encode(src), host.new_cache(), 0)
    got = dev.decode_step(dec, dev.encode(src), dev.new_cache(), 0)
    _close(got, want, 5e-2, 5e-2)
    out = dev.translate([10, 11, 12, 13, 2], 20, num_beams=3, max_new_tokens=8)
    assert len(out) <= 8 and all(0 <= x < 512 for x in out)


def test_nvfp4_experts_take_the_grouped_gemm_on_128_row_aligned_segments():
    """NVFP4 MoE checkpoints: the expert sort pads every expert's rows to the 128-row tile of the scale factors and
    the grouped tcgen05 GEMM takes the W4A4 operands. Checked three ways: against one GEMM per active expert on the
    same device (same quantisation, so the two agree closely), against the CPU restatement of the same synthetic
    checkpoint, and end to end with CUDA graphs on."""
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.models.moe import moe_block, routed_experts
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.models.decoder import Decoder
    from metrale_inference_alpha_b200.ops import ACT_FOR_WEIGHT
    from metrale_inference_alpha_b200.weights.loader import load_weights
    from metrale_inference_alpha_b200.weights.source import SyntheticSource
    cfg = preset("tiny-hybrid-moe", weight_format="nvfp4")
    # the same synthetic checkpoint on both devices
    w_h = load_weights(cfg, SyntheticSource(cfg, seed=3, device="cpu"), device="cpu")
    w_d = load_weights(cfg, SyntheticSource(cfg, seed=3, device="cpu"), device=DEV)
    lw_d = next(L for L in w_d.layers if L.ffn_kind == "moe")
    lw_h = next(L for L in w_h.layers if L.ffn_kind == "moe")
    assert lw_d.ffn.grouped is not None and lw_d.ffn.grouped.gate_up.fmt == "nvfp4"
    fmt = ACT_FOR_WEIGHT["nvfp4"]
    dh, dd = Decoder(cfg, w_h, device="cpu"), Decoder(cfg, w_d, device=DEV)
    E, K = cfg.num_experts, cfg.experts_per_token
    for T in (3, 24, 300):                     # 300 x 2 pairs over 8 experts: some experts span several 128-row tiles
        g = torch.Generator().manual_seed(15 + T)
        x = (torch.randn(T, cfg.hidden_size, generator=g)).to(torch.bfloat16)
        # the same routing on every side (a near-tie in the router would send a token to different experts)
        idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
        if T == 3:
            idx[:, 0] = 5                      # most experts empty
        wts = torch.rand(T, K, generator=g)
        a_d = dd._norm_act(x.to(DEV), lw_d.ln2, fmt, also_bf16=True)
        got = routed_experts(dd, a_d, wts.to(DEV), idx.to(DEV), lw_d.ffn).float().cpu()
        grouped, lw_d.ffn.grouped = lw_d.ffn.grouped, None
        try:
            each = routed_experts(dd, a_d, wts.to(DEV), idx.to(DEV), lw_d.ffn).float().cpu()
        finally:
            lw_d.ffn.grouped = grouped
        assert torch.isfinite(got).all()
        scale = float(each.abs().mean())
        # the grouped path gathers the 4-bit rows the norm produced, the per-expert path re-quantises their bf16
        # copy with scales of its own: the two agree within the format's noise
        assert float((got - each).abs().mean()) < 0.2 * scale, (T, float((got - each).abs().mean()), scale)
        a_h = dh._norm_act(x, lw_h.ln2, fmt, also_bf16=True)
        want = routed_experts(dh, a_h, wts, idx, lw_h.ffn).float()
        err = (got - want).abs()
        # host and device round the 4-bit activations independently, so they agree within the format's noise
        # (a wrong expert or scale would be off by ~100 %)
        assert float(err.mean()) < 0.2 * float(want.abs().mean()), (T, float(err.mean()), float(want.abs().mean()))
    assert moe_block(dd, x.to(DEV), lw_d).shape == x.shape
    eng = LLMEngine(EngineArgs(model=cfg, device=DEV, num_kv_blocks=64, max_num_seqs=4))
    assert eng.args.use_cuda_graphs
    out = eng.generate([list(range(5, 40))], SamplingParams(max_tokens=4, temperature=0.0))[0]
    assert len(out.output_ids) == 4
    ops.check_status(torch.device(DEV))


def test_expert_sort_with_aligned_tiles_marks_every_empty_row():
    from metrale_inference_alpha_b200.ops.moe_cuda import SortedPairs
    g = torch.Generator().manual_seed(4)
    T, K, E = 77, 3, 6
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    idx[idx == 4] = 5                                     # expert 4 gets nothing (and 5 may repeat in a row)
    flat = idx.view(-1)
    for tr in (128, 32):                                  # every tile starts a 128-row slot and fills its first `tr` rows
        sp = SortedPairs(idx.to(DEV), 1, 5, tr, align=128)    # local experts 1..5; expert 0's pairs are not local
        torch.cuda.synchronize()
        off = sp.expert_off.cpu().tolist()
        total = int(sp.total_rows.item())
        row_pair = sp.row_pair.cpu()
        pair_row = sp.pair_row.cpu().view(-1)
        assert all(o % 128 == 0 for o in off) and off[-1] == total and total <= sp.rows_cap == row_pair.numel()
        live_rows = []
        for e in range(5):
            n = int((flat == e + 1).sum())
            assert off[e + 1] - off[e] == (n + tr - 1) // tr * 128
            live_rows += [off[e] + (i // tr) * 128 + i % tr for i in range(n)]
            assert (flat[row_pair[live_rows[len(live_rows) - n:]].long()] == e + 1).all()
        mask = torch.zeros(sp.rows_cap, dtype=torch.bool)
        mask[live_rows] = True
        assert (row_pair[mask] >= 0).all() and (row_pair[~mask] == -1).all()
        assert (pair_row[flat == 0] == -1).all()
        live = pair_row[flat != 0].long()
        assert (row_pair[live] == torch.nonzero(flat != 0).view(-1)).all()
        tiles = [(int(e), int(r0), int(n)) for e, r0, n in zip(sp.tile_expert.cpu(), sp.tile_row0.cpu(), sp.tile_nrows.cpu()) if e >= 0]
        assert all(r0 % 128 == 0 and 0 < n <= tr for _, r0, n in tiles)
        assert sum(n for _, _, n in tiles) == int((flat != 0).sum())


def test_kernel_audit_shows_which_kernels_served_a_long_prefill_and_a_decode_step():
    from metrale_inference_alpha_b200.engine.llm_engine import EngineArgs, LLMEngine
    from metrale_inference_alpha_b200.sampling.params import SamplingParams
    from metrale_inference_alpha_b200.utils.kernel_audit import KernelAudit
    eng = LLMEngine(EngineArgs(model="tiny-hybrid-moe", device=DEV, num_kv_blocks=64, max_num_seqs=2, use_cuda_graphs=False))
    with KernelAudit() as audit:
        eng.generate([list(range(5, 5 + 200))], SamplingParams(max_tokens=3, temperature=0.0))
    res = audit.resolve()
    # a 200-token prefill takes the chunked gated-delta-rule scan, the time-parallel conv and the tcgen05 attention
    audit.require("gdn_chunked")
    audit.require("causal_conv1d_par")
    audit.require("attn_prefill_tc")
    assert res["gemm"]["gemm"] > 10 and "moe routing" in res and "sampling" in res
    assert res["gated delta rule"].get("gdn_recurrence", 0) > 0          # the decode steps
    with pytest.raises(AssertionError):
        audit.require("kda_recurrence")
    with pytest.raises(AssertionError):
        audit.require("gemm", never=["row_op"])


@pytest.mark.parametrize("fused_norm", [False, True])
def test_kda_chunked_prefill_matches_the_token_recurrence(fused_norm, monkeypatch):
    """Long rows take the chunked kernels; forcing the token-by-token kernel on the same inputs must give the
    same outputs and the same final state: a fresh 200-token sequence, a 130-token continuation of an existing
    state and a 7-token sequence in one ragged batch."""
    g = torch.Generator().manual_seed(16)
    H, D = 3, 128
    lens, starts = [200, 130, 7], [0, 40, 0]
    T = sum(lens)
    conv = torch.randn(T, 3 * H * D, generator=g)
    g_raw = torch.randn(T, H * D, generator=g) * 2
    b_raw = torch.randn(T, H + 2, generator=g)[:, :H]                  # a strided beta view
    A_log, dtb = torch.randn(H, generator=g) * 0.3, torch.randn(H * D, generator=g) * 0.3
    st = torch.randn(5, H, D, D, generator=g) * 0.1
    gate = torch.randn(T, H * D, generator=g).to(torch.bfloat16)
    w = torch.rand(D, generator=g) + 0.5
    seqs = [dict(tokens=[1] * n, start_pos=s, blocks=list(range(1, 20)), state_slot=i + 1) for i, (n, s) in enumerate(zip(lens, starts))]
    b = ForwardBatch.build(seqs, 16, device=DEV)
    outs = {}
    for name, thresh in (("chunked", 64), ("sequential", 1 << 30)):
        monkeypatch.setattr(rops, "_KDA_CHUNK_MIN_TOKENS", thresh)
        s = st.clone().to(DEV)
        norm = (w.to(DEV), gate.to(DEV), 1e-6) if fused_norm else None
        with ops._native.launch_trace() as names:
            y = rops.kda_recurrence(conv.to(DEV), g_raw.to(DEV), b_raw.to(DEV), A_log.to(DEV), dtb.to(DEV), -5.0, s, b,
                                    heads=H, dim=D, norm=norm)
        assert ("kda_chunked" in names) == (name == "chunked")
        outs[name] = (y.float().cpu(), s.cpu())
    tol = 2e-2 if fused_norm else 2e-3
    _close(outs["chunked"][0], outs["sequential"][0], tol, tol)
    _close(outs["chunked"][1], outs["sequential"][1], 2e-3, 2e-3)
    assert torch.equal(outs["chunked"][1][0], st[0]) and torch.equal(outs["chunked"][1][4], st[4])       # untouched slots
    ops.check_status(torch.device(DEV))
