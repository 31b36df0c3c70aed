"""Executes step plans on one device: stages the step's metadata through pinned host memory
into fixed device buffers, runs the decoder (a CUDA graph per batch rung for decode, eager for
prefill / verify), selects tokens on the device and reads back 4 bytes per sampled row.

Role of the reference's ``TransformerModel`` forward entry points
(``crates/model-engine/src/model/trait_impl/decode_a2.rs``: rung padding, fixed-address
metadata, graph cache; ``prefill_b.rs``: chunked prefill; ``verify_e.rs``: batched verify;
``meta_argmax.rs``: device argmax + 4*n-byte readback) and of ``factory/build.rs`` (KV budget).
"""
from __future__ import annotations

import contextlib
import gc
import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import ops
from ..utils import nvtx
from ..cache import KvCacheConfig, PagedKvCache, StatePool
from ..config.model_config import ModelConfig
from ..models.decoder import Decoder, LayerCaches, TpContext
from ..scheduler.policy import SchedulerConfig
from ..scheduler.types import StepPlan, StepResult
from ..weights.loader import ModelW
from .batch import ForwardBatch


def state_shapes(cfg: ModelConfig, w: ModelW):
    """(conv window, ssm matrix) shapes of every recurrent layer, from the loaded (sharded) weights."""
    out = []
    for lw in w.layers:
        if lw.kind == "gdn":
            m = lw.mixer
            C = 2 * m.k_heads * cfg.gdn_k_dim + m.v_heads * cfg.gdn_v_dim
            out.append(((C, cfg.conv_kernel - 1), (m.v_heads, cfg.gdn_k_dim, cfg.gdn_v_dim)))
        elif lw.kind == "kda":
            m = lw.mixer
            out.append(((3 * m.heads * cfg.kda_head_dim, cfg.conv_kernel - 1), (m.heads, cfg.kda_head_dim, cfg.kda_head_dim)))
        elif lw.kind == "mamba2":
            m = lw.mixer
            C = m.heads * cfg.mamba_head_dim + 2 * m.groups * cfg.mamba_state
            out.append(((C, cfg.conv_kernel - 1), (m.heads, cfg.mamba_head_dim, cfg.mamba_state)))
    return out


def kv_config(cfg: ModelConfig, w: ModelW, block_size: int, mtp: bool = False) -> KvCacheConfig:
    if cfg.arch == "deepseek_mla":
        # with a sparse-attention indexer, the pool's second tensor holds the indexer key of every token
        return KvCacheConfig(1 if mtp else len(cfg.attention_layers()), 1, cfg.kv_lora_rank + cfg.qk_rope_dim,
                             block_size, cfg.kv_dtype if cfg.kv_dtype == "bf16" else "bf16",
                             v_head_dim=cfg.index_head_dim if cfg.index_topk > 0 else None, has_v=cfg.index_topk > 0)
    kvh = cfg.num_kv_heads
    for lw in ([w.mtp.layer] if (mtp and w.mtp) else w.layers):
        if lw.kind == "attention":
            kvh = lw.mixer.kv_heads
            break
    att = cfg.attention_layers()
    hp = () if mtp else tuple(i for i, layer in enumerate(att) if layer in set(cfg.kv_high_precision_layers))
    return KvCacheConfig(1 if mtp else max(1, len(att)), kvh, cfg.head_dim, block_size, cfg.kv_dtype,
                         high_precision_layers=hp)


@contextlib.contextmanager
def _capture(g: "torch.cuda.CUDAGraph"):
    """Stream capture that other activity in the process cannot invalidate: the capture-error mode is
    thread-local (HTTP handler threads, samplers and exporters may call into CUDA while the scheduler
    thread captures), and Python's cyclic collector is held off for the duration (a collection inside
    the capture could free pinned staging buffers of retired engines, which is not a capturable
    operation)."""
    was = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            yield
    finally:
        if was:
            gc.enable()


class _Stager:
    """One pinned int32 buffer + one device int32 buffer; a step's integer metadata crosses
    PCIe in a single async copy of just the bytes in use. The field layout is a function of
    (token capacity, sequence capacity), so a CUDA-graph rung always sees the same addresses."""

    FIELDS = ("slots", "tokens", "pos", "q_start", "q_len", "ctx", "state", "lrows", "bt")

    def __init__(self, max_tokens: int, max_seqs: int, max_blocks: int, device):
        self.max_tokens, self.max_seqs, self.max_blocks = max_tokens, max_seqs, max_blocks
        self.device = torch.device(device)
        self.total = self._layout(max_tokens, max_seqs)[1]
        pin = self.device.type == "cuda"
        self.host = torch.zeros(self.total, dtype=torch.int32, pin_memory=pin)
        self.np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=self.device)
        self.bytes_per_copy = 0
        self.off = {}
        self.used = 0
        # the async H2D copy reads the pinned buffer when the stream gets to it, not when it is
        # enqueued: the event marks that point, and nothing rewrites the buffer before it
        self.copied = torch.cuda.Event() if pin else None
        self.in_flight = False

    def _layout(self, T: int, S: int):
        off, o = {}, 0
        # token ids come first so that an upload can leave them out (look-ahead decode: the device
        # wrote them itself); every field starts on an even offset, which keeps the int64 fields
        # (slot_mapping, logit rows) 8-byte aligned
        for name, n in (("tokens", T), ("slots", 2 * T), ("lrows", 2 * T), ("pos", T), ("q_start", S),
                        ("q_len", S), ("ctx", S), ("state", S), ("bt", S * self.max_blocks)):
            off[name] = (o, n)
            o += n + (n & 1)
        return off, o

    def wait_copied(self) -> None:
        """Block until the last upload has read the pinned buffer (call before rewriting it)."""
        if self.in_flight:
            self.copied.synchronize()
            self.in_flight = False

    def begin(self, T_cap: int, S_cap: int) -> None:
        assert T_cap <= self.max_tokens and S_cap <= self.max_seqs, (T_cap, S_cap)
        self.wait_copied()
        self.off, self.used = self._layout(T_cap, S_cap)
        self.S_cap = S_cap

    def view(self, buf, name, n=None):
        o, cap = self.off[name]
        return buf[o:o + (cap if n is None else n)]

    def upload(self, skip_tokens: bool = False) -> None:
        lo = self.off["slots"][0] if skip_tokens else 0
        self.dev[lo:self.used].copy_(self.host[lo:self.used], non_blocking=True)
        self.bytes_per_copy = (self.used - lo) * 4
        if self.copied is not None:
            self.copied.record()
            self.in_flight = True


class ModelRunner:
    def __init__(self, cfg: ModelConfig, weights: ModelW, device="cpu", num_blocks: int = 256,
                 sched: Optional[SchedulerConfig] = None, tp: Optional[TpContext] = None,
                 use_graphs: bool = True, max_state_slots: Optional[int] = None, num_snapshots: int = 16,
                 mtp_drafts: int = 0, kv_poison: bool = False, fp8_kv_calibration_tokens: int = 0,
                 fp8_kv_headroom: float = 1.0):
        self.cfg, self.w, self.device = cfg, weights, torch.device(device)
        self.sched = sched or SchedulerConfig()
        self.tp = tp or TpContext()
        bs = self.sched.block_size
        self.block_size = bs
        self.kv = PagedKvCache(kv_config(cfg, weights, bs), num_blocks, device, poison=kv_poison)
        self.mtp_kv = None
        if weights.mtp is not None:
            self.mtp_kv = PagedKvCache(kv_config(cfg, weights, bs, mtp=True), num_blocks, device)
        shapes = state_shapes(cfg, weights)
        self.pool = None
        if shapes:
            slots = (max_state_slots or self.sched.max_num_seqs) + 1
            self.pool = StatePool(shapes, slots, num_snapshots, device)
        self.caches = LayerCaches(cfg, kv=self.kv, state=self.pool, mtp_kv=self.mtp_kv)
        self.decoder = Decoder(cfg, weights, self.tp, device)
        self.dflash = None
        # FP8 KV scales: the checkpoint's (three key spellings, weights/kv_scales.py), else online
        # calibration over the first tokens when asked for, else 1.0
        self.kv_scales_loaded = 0
        att = [lw for lw in weights.layers if lw.kind == "attention"]
        for j, lw in enumerate(att):
            sc = getattr(lw.mixer, "kv_scale", None)
            if sc is not None and j < len(self.kv.k_scale) and self.kv.k[j].dtype == torch.uint8:
                self.kv.k_scale[j].fill_(sc[0])
                self.kv.v_scale[j].fill_(sc[1])
                self.kv_scales_loaded += 1
        self.kv_cal = None
        if fp8_kv_calibration_tokens > 0 and self.kv_scales_loaded == 0 and cfg.arch != "deepseek_mla":
            from ..cache.fp8_calibration import Fp8KvCalibration
            cal = Fp8KvCalibration(self.kv, fp8_kv_calibration_tokens, fp8_kv_headroom)
            if not cal.frozen:
                self.kv_cal = self.decoder.kv_cal = cal
        self.max_blocks = (self.sched.max_model_len + bs - 1) // bs
        self.max_seqs = max(self.sched.batch_rungs[-1], self.sched.max_num_seqs)
        max_tokens = max(self.sched.max_prefill_tokens + self.max_seqs, self.max_seqs * 8)
        self.stage = _Stager(max_tokens, self.max_seqs, self.max_blocks, device)
        if hasattr(self.tp, "setup_fused") and self.device.type == "cuda":
            self.tp.setup_fused(cfg.hidden_size, max_tokens)         # collective: symmetric buffers of the fused reduction
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self.graphs: Dict[Tuple, object] = {}
        self.mtp_drafts = mtp_drafts if weights.mtp is not None else 0
        S = max_tokens                   # one entry per sampled row (verify rows included)
        dev = self.device
        # sampling parameters, fixed addresses
        self.s_temp = torch.zeros(S, dtype=torch.float32, device=dev)
        self.s_topk = torch.zeros(S, dtype=torch.int32, device=dev)
        self.s_topp = torch.ones(S, dtype=torch.float32, device=dev)
        self.s_minp = torch.zeros(S, dtype=torch.float32, device=dev)
        self.s_seed = torch.zeros(S, dtype=torch.int64, device=dev)
        self.s_step = torch.zeros(S, dtype=torch.int64, device=dev)
        self.out_ids = torch.zeros(max_tokens, dtype=torch.int32, device=dev)
        self.out_lp = torch.zeros(max_tokens, dtype=torch.float32, device=dev)
        pin = dev.type == "cuda"
        self.host_ids = torch.zeros(max_tokens, dtype=torch.int32, pin_memory=pin)
        self.host_lp = torch.zeros(max_tokens, dtype=torch.float32, pin_memory=pin)
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        # the kernels' status word (expired bounded waits, out-of-range indices that skipped an
        # access) rides back with the sampled ids: no extra synchronisation
        self.host_status = torch.zeros(4, dtype=torch.int32, pin_memory=pin)
        self.status_pending = False
        self.last_hidden = None
        self.graph_replays = 0
        self.logit_processor = None    # fn(seq, row_logits fp32 [V]) -> row_logits, host-logits path

    # ------------------------------------------------------------------ batch staging
    def _stage_decode_incremental(self, plan: StepPlan, pad_seqs: int, ahead: bool = False) -> bool:
        """Plain decode of the same sequences as the previous staged decode step: the pinned
        staging arrays still hold that step, so advance them in place (vectorised: positions and
        context + 1, slots recomputed from the block table, block-table entries only for the
        sequences that crossed into a new block) instead of rebuilding every row in Python."""
        st, bs, items = self.stage, self.block_size, plan.items
        S = len(items)
        sig = (pad_seqs, tuple(it.seq.seq_id for it in items))
        if sig != self._fast_sig:
            self._fast_sig_next = sig
            return False
        npv = lambda name: st.view(st.np, name)
        pos, ctx, tokens = npv("pos"), npv("ctx"), npv("tokens")
        if items[0].start_pos != pos[0] + 1 or items[-1].start_pos != pos[S - 1] + 1:
            self._fast_sig_next = sig
            return False
        st.wait_copied()
        if not ahead:                                         # look-ahead: the previous step's argmax fed them on the device
            tokens[:S] = [it.tokens[0] for it in items]
        pos[:S] += 1
        ctx[:S] += 1
        p = pos[:S]
        bt2 = npv("bt").reshape(st.S_cap, st.max_blocks)
        for s in np.nonzero(p % bs == 0)[0]:
            bt2[s, p[s] // bs] = items[s].seq.blocks[p[s] // bs]
        slots = npv("slots").view(np.int64)
        slots[:S] = bt2[np.arange(S), p // bs].astype(np.int64) * bs + p % bs
        st.upload(skip_tokens=ahead)
        self.h2d_bytes += st.bytes_per_copy
        return True

    def _stage(self, plan: StepPlan, pad_seqs: int = 0, logits_all_verify: bool = True, pad_q: int = 1) -> ForwardBatch:
        """`pad_seqs`: pad with null sequences (rows that write nothing) up to this many, each of
        `pad_q` rows, so that a CUDA-graph rung always sees the same layout."""
        st, bs = self.stage, self.block_size
        self._fast_sig, self._fast_sig_next = None, None      # any full staging invalidates the fast path
        n_rows = sum(len(i.tokens) for i in plan.items)
        n_seqs = max(len(plan.items), pad_seqs)
        pad_rows = max(0, pad_seqs - len(plan.items)) * pad_q
        if pad_seqs:
            st.begin(n_rows + pad_rows, n_seqs)               # graph rung: exact, fixed layout
        else:
            st.begin(min(st.max_tokens, (n_rows + 63) // 64 * 64), min(st.max_seqs, (n_seqs + 7) // 8 * 8))
        npv = lambda name: st.view(st.np, name)
        tokens, pos, qs, ql, ctx, state, bt = (npv(n) for n in ("tokens", "pos", "q_start", "q_len", "ctx", "state", "bt"))
        slots = npv("slots").view(np.int64)
        lrows = npv("lrows").view(np.int64)
        bt2 = bt.reshape(st.S_cap, st.max_blocks)
        row = 0
        nl = 0
        max_q = 1
        max_ctx = 1
        for s, it in enumerate(plan.items):
            n = len(it.tokens)
            p0 = it.start_pos
            tokens[row:row + n] = it.tokens
            pos[row:row + n] = np.arange(p0, p0 + n, dtype=np.int32)
            blocks = it.seq.blocks
            nb = len(blocks)
            bt2[s, :nb] = blocks
            pp = np.arange(p0, p0 + n)
            barr = np.asarray(blocks, dtype=np.int64)
            slots[row:row + n] = barr[pp // bs] * bs + pp % bs
            qs[s], ql[s], ctx[s], state[s] = row, n, p0 + n, it.seq.state_slot
            if it.sample:
                k = it.verify if logits_all_verify else 0
                lrows[nl:nl + k + 1] = np.arange(row + n - 1 - k, row + n)
                nl += k + 1
            row += n
            max_q, max_ctx = max(max_q, n), max(max_ctx, p0 + n)
        S = len(plan.items)
        while S < pad_seqs:                                   # null rows up to the graph rung
            tokens[row:row + pad_q], slots[row:row + pad_q] = 0, -1
            pos[row:row + pad_q] = np.arange(pad_q, dtype=np.int32)
            qs[S], ql[S], ctx[S], state[S] = row, pad_q, pad_q, 0
            bt2[S, 0] = 0
            lrows[nl:nl + pad_q] = np.arange(row, row + pad_q)
            nl += pad_q
            row += pad_q
            S += 1
            max_q = max(max_q, pad_q)
        st.upload()
        self.h2d_bytes += st.bytes_per_copy
        dv = lambda name, n: st.view(st.dev, name, n)
        b = ForwardBatch(
            token_ids=dv("tokens", row), positions=dv("pos", row),
            slot_mapping=dv("slots", 2 * row).view(torch.int64),
            q_start=dv("q_start", S), q_len=dv("q_len", S), ctx_len=dv("ctx", S),
            block_table=dv("bt", None).view(st.S_cap, st.max_blocks)[:S],
            logit_rows=dv("lrows", 2 * nl).view(torch.int64),
            max_q_len=max_q, max_ctx=max_ctx, state_slots=dv("state", S), num_tokens=row, num_seqs=S)
        return b

    _fast_sig = None
    _fast_sig_next = None

    # ------------------------------------------------------------------ static activation scales
    def calibrate_static_scales(self, tokens: int = 256, margin: float = 2.0, seed: int = 1234) -> int:
        """NVFP4 models: fix the global scale of the down projection's and o projection's input per layer (what a
        ModelOpt checkpoint calls `input_scale`), so that the quantiser becomes row-local and can
        run inside the producing GEMM's epilogue. One prefill of random tokens through temporary
        KV blocks records max |SwiGLU output| per layer; scale = margin * amax / (6 * 448).
        Checkpoint-provided scales (already > 0) are kept. Returns the number of layers set."""
        ffns = [lw.ffn for lw in self.w.layers
                if lw.ffn_kind == "dense" and getattr(lw.ffn, "interleaved", False) and lw.ffn.down.fmt == "nvfp4"]
        attns = [lw.mixer for lw in self.w.layers
                 if lw.kind == "attention" and lw.mixer.o.fmt == "nvfp4" and not self.cfg.attn_output_gate]
        todo = [f for f in ffns if f.down_in_scale <= 0.0]
        todo_a = [m for m in attns if m.o_in_scale <= 0.0]
        if not todo and not todo_a:
            for f in ffns:
                ops.static_scale_vec(self.device, f.down_in_scale, 256)
            for m in attns:
                ops.static_scale_vec(self.device, m.o_in_scale, 256)
            return 0
        tokens = min(tokens, self.sched.max_prefill_tokens, self.sched.max_model_len - 1)
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(1, self.cfg.vocab_size, (tokens,), generator=g).tolist()
        nblk = (tokens + self.block_size - 1) // self.block_size
        blocks = self.kv.allocator.alloc(nblk)
        try:
            batch = ForwardBatch.build([dict(tokens=ids, start_pos=0, blocks=blocks, state_slot=0, logits="none")],
                                       self.block_size, device=self.device, max_blocks=self.max_blocks)
            self.decoder.calib = {}
            kv_cal, self.decoder.kv_cal = self.decoder.kv_cal, None      # random tokens must not count towards the KV scales
            self.decoder.backbone(batch, self.caches)
            self.tp.end_forward()
            calib = self.decoder.calib
        finally:
            self.decoder.calib = None
            self.decoder.kv_cal = self.kv_cal
            self.kv.allocator.free(blocks)
        n = 0
        for f in todo:
            if id(f) in calib:
                amax = float(calib[id(f)])
                if amax > 0.0:
                    f.down_in_scale = margin * amax / (6.0 * 448.0)
                    n += 1
        for m in todo_a:
            if id(m) in calib:
                amax = float(calib[id(m)])
                if amax > 0.0:
                    m.o_in_scale = margin * amax / (6.0 * 448.0)
        for f in ffns:
            if f.down_in_scale > 0.0:
                ops.static_scale_vec(self.device, f.down_in_scale, 256)
        for m in attns:
            if m.o_in_scale > 0.0:
                ops.static_scale_vec(self.device, m.o_in_scale, 256)
        return n

    def _adapter_rows(self, plan: StepPlan) -> Optional[torch.Tensor]:
        """Adapter slot of every token row of the step, or None when no sequence uses an adapter."""
        lora = self.decoder.lora
        if lora is None or not any(i.seq.req.adapter for i in plan.items):
            return None
        rows: List[int] = []
        for it in plan.items:
            rows += [lora.slot_of(it.seq.req.adapter)] * len(it.tokens)
        cap = (len(rows) + 63) // 64 * 64
        rows += [-1] * (cap - len(rows))
        t = torch.tensor(rows, dtype=torch.int32)
        self.h2d_bytes += t.numel() * 4
        return t.to(self.device, non_blocking=True)

    def _stage_with_adapters(self, plan: StepPlan) -> ForwardBatch:
        batch = self._stage(plan)
        batch.adapter_rows = self._adapter_rows(plan)
        if any(i.seq.req.mm is not None for i in plan.items):
            self._attach_multimodal(plan, batch)
        self.pending_stash = None
        if self.pool is not None and any(i.verify for i in plan.items):
            from .batch import SpecStash
            batch.spec_stash = self.pending_stash = SpecStash(batch)
        return batch

    pending_stash = None

    def _attach_multimodal(self, plan: StepPlan, batch: ForwardBatch) -> None:
        """Steps that hold a sequence with images: rows on placeholder tokens take the vision tower's
        embeddings, and every row gets its rotary row from three-axis positions (prompt rows from the
        request's index, generated rows from sequence index + the request's offset on all axes)."""
        from ..vision.mrope import gather_tables
        dec = self.decoder
        T = batch.num_tokens
        pos3 = torch.zeros(3, T, dtype=torch.int64)
        rows, embs = [], []
        r = 0
        for it in plan.items:
            n, p0, mm = len(it.tokens), it.start_pos, it.seq.req.mm
            idx = torch.arange(p0, p0 + n)
            if mm is None:
                pos3[:, r:r + n] = idx
            else:
                L = mm.positions.shape[1]
                inside = idx < L
                pos3[:, r:r + n] = torch.where(inside, mm.positions[:, idx.clamp(max=L - 1)], idx + mm.delta)
                for j in range(n):
                    e = mm.row_of_token.get(p0 + j)
                    if e is not None:
                        rows.append(r + j)
                        embs.append(e)
            r += n
        half = dec.cos.shape[1]
        sections = self.cfg.mrope_sections or [half - 2 * (half // 3), half // 3, half // 3]
        cos, sin = gather_tables(dec.cos, dec.sin, pos3[:, :T].to(self.device), sections)
        pad = batch.token_ids.shape[0] - T
        if pad > 0:
            cos = torch.cat([cos, cos.new_ones(pad, half)])
            sin = torch.cat([sin, sin.new_zeros(pad, half)])
        batch.rope_tables = (cos.contiguous(), sin.contiguous())
        batch.rope_rows = torch.arange(batch.token_ids.shape[0], dtype=torch.int32, device=self.device)
        if rows:
            mmv = [it.seq.req.mm for it in plan.items if it.seq.req.mm is not None]
            table = torch.cat([m.embeds for m in mmv], 0)
            base, off = {}, 0
            for m in mmv:
                base[id(m)] = off
                off += m.embeds.shape[0]
            sel = []
            r = 0
            for it in plan.items:
                mm = it.seq.req.mm
                if mm is not None:
                    for j in range(len(it.tokens)):
                        e = mm.row_of_token.get(it.start_pos + j)
                        if e is not None:
                            sel.append(base[id(mm)] + e)
                r += len(it.tokens)
            batch.embed_override = (torch.tensor(rows, dtype=torch.int64, device=self.device),
                                    table[torch.tensor(sel, dtype=torch.int64, device=self.device)])
            self.h2d_bytes += 16 * len(rows)

    def commit_recurrent(self, plan: StepPlan) -> None:
        """After the scheduler has applied a verify step: advance the recurrent state of every
        sequence by the rows it accepted (the verify forward left the state untouched)."""
        stash, self.pending_stash = self.pending_stash, None
        if stash is None:
            return
        import dataclasses
        from ..models.recurrent import commit_recurrent
        b = stash.batch
        n = [0] * b.q_len.numel()
        for s, it in enumerate(plan.items):
            if it.seq.is_finished():
                continue
            n[s] = (getattr(it.seq, "last_accept", 0) + 1) if it.verify else len(it.tokens)
        ql = torch.tensor(n, dtype=torch.int32)
        self.h2d_bytes += ql.numel() * 4
        cb = dataclasses.replace(b, q_len=ql.to(self.device, non_blocking=True), spec_stash=None)
        commit_recurrent(self.cfg, self.pool, stash, cb)

    def _set_sampling(self, plan: StepPlan) -> bool:
        """Upload per-row sampling parameters (one entry per sampled row: a sequence that verifies
        k drafts contributes k + 1 rows; drafts are only ever given to greedy sequences, whose rows
        carry temperature 0 and are selected by argmax inside the sampler). Returns True when every
        row is greedy."""
        all_greedy = all(i.seq.req.params.greedy for i in plan.items)
        if all_greedy:
            return True
        items = [i for i in plan.items if i.sample for _ in range(i.verify + 1)]
        n = len(items)
        P = [i.seq.req.params for i in items]
        dev = self.device
        self.s_temp[:n] = torch.tensor([p.temperature for p in P], dtype=torch.float32).to(dev, non_blocking=True)
        self.s_topk[:n] = torch.tensor([p.top_k for p in P], dtype=torch.int32).to(dev, non_blocking=True)
        self.s_topp[:n] = torch.tensor([p.top_p for p in P], dtype=torch.float32).to(dev, non_blocking=True)
        self.s_minp[:n] = torch.tensor([p.min_p for p in P], dtype=torch.float32).to(dev, non_blocking=True)
        seeds = [(p.seed if p.seed is not None else i.seq.seq_id * 1000003) & ((1 << 62) - 1)
                 for p, i in zip(P, items)]
        self.s_seed[:n] = torch.tensor(seeds, dtype=torch.int64).to(dev, non_blocking=True)
        self.s_step[:n] = torch.tensor([i.seq.sample_step for i in items], dtype=torch.int64).to(dev, non_blocking=True)
        self.h2d_bytes += n * 32
        return False

    def _after_forward(self, batch: ForwardBatch) -> None:
        """Per-forward bookkeeping that is not part of the model: the collective epilogue and the
        FP8 KV scale calibration window."""
        self.tp.end_forward()
        if self.kv_cal is not None and self.kv_cal.after_step(batch.slot_mapping):
            self.kv_cal = self.decoder.kv_cal = None          # frozen: graphs may be used from now on

    def graphs_ready(self) -> bool:
        """CUDA graphs stay off while the KV scales are still being calibrated."""
        return self.use_graphs and self.kv_cal is None

    # ------------------------------------------------------------------ device status
    def _post_status(self) -> None:
        """Queue a copy of the status word behind the step's kernels."""
        if self.device.type == "cuda":
            self.host_status.copy_(ops.runtime(self.device).status, non_blocking=True)
            self.status_pending = True
            self.d2h_bytes += 16

    def _check_status(self) -> None:
        """After a stream synchronisation: raise if any kernel since the last check reported."""
        if not self.status_pending:
            return
        self.status_pending = False
        code = int(self.host_status[0])
        if code:
            if self.device.type == "cuda":
                ops.runtime(self.device).status.zero_()
            from ..ops._native import KernelError
            what = {0x400: "a peer wait expired", 0x500: "an out-of-range index skipped an access"}.get(
                code, "a bounded wait expired")
            raise KernelError(f"device status 0x{code:x}: {what}")

    # ------------------------------------------------------------------ forward variants
    def _forward_select(self, batch: ForwardBatch, greedy: bool, want_lp: bool, n_rows: int, feed: bool = False):
        """decoder forward + on-device token selection into self.out_ids[:n_rows]. `feed`: greedy
        selection also writes each id into the batch's own token buffer, the next decode step's
        input (look-ahead decode)."""
        feed_t = batch.token_ids[:n_rows] if (feed and greedy and not want_lp) else None
        merge = greedy and not want_lp and getattr(self.tp, "reduce", None) is not None
        logits, hidden = self.decoder.forward(batch, self.caches, out_f32=not greedy, gather_logits=not merge)
        self.last_hidden = hidden
        if merge:
            # vocabulary-parallel greedy selection: one (max, index) pair per rank and row crosses NVLink
            self.tp.reduce.argmax_merge(logits, self.w.vocab_lo, self.out_ids[:n_rows], feed_t)
        elif greedy:
            if want_lp:
                _, lp = ops.argmax(logits, logprob=True, out=self.out_ids[:n_rows])
                self.out_lp[:n_rows].copy_(lp)
            else:
                ops.argmax(logits, out=self.out_ids[:n_rows], feed=feed_t)
        else:
            ids, lp = ops.sample(logits, self.s_temp[:n_rows], self.s_topk[:n_rows], self.s_topp[:n_rows],
                                 self.s_minp[:n_rows], self.s_seed[:n_rows], self.s_step[:n_rows])
            self.out_ids[:n_rows].copy_(ids)
            self.out_lp[:n_rows].copy_(lp)
        self._after_forward(batch)
        return logits

    def _rung(self, n: int) -> int:
        for r in self.sched.batch_rungs:
            if n <= r:
                return r
        return n

    def _decode_graph(self, plan: StepPlan, greedy: bool, want_lp: bool, ahead: bool = False):
        """Replay (capturing on first use) the CUDA graph for this batch rung. `ahead`: the step's
        tokens are already in the device buffer (fed by the previous step); returns None when such
        a step cannot be staged incrementally."""
        n = len(plan.items)
        rung = self._rung(n)
        key = (rung, greedy, want_lp)
        if key not in self.graphs:
            # warm-up + capture on an all-null batch (rows that write nothing and touch only
            # the scratch state slot), so capturing never advances a live sequence
            null = self._stage(StepPlan("decode", []), pad_seqs=rung)
            null.max_ctx, null.max_q_len = self.sched.max_model_len, 1   # fixed launch geometry
            self._forward_select(null, greedy, want_lp, rung, feed=True)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            count0 = ops.launch_count
            with _capture(g):
                self._forward_select(null, greedy, want_lp, rung, feed=True)
            self.graphs[key] = (g, ops.launch_count - count0, self.last_hidden)
        if not self._stage_decode_incremental(plan, rung, ahead):
            if ahead:
                return None
            sig = self._fast_sig_next
            self._stage(plan, pad_seqs=rung)
            self._fast_sig = sig                              # the arrays now hold this decode step
        g, launches, hidden = self.graphs[key]
        g.replay()
        ops.launch_count += launches
        self.graph_replays += 1
        self.last_hidden = hidden
        return rung

    def _verify_graph(self, plan: StepPlan, K: int) -> None:
        """Replay (capturing on first use) the CUDA graph of a speculative verify step in which
        every sequence feeds K drafts: one forward over rung x (K + 1) rows, argmax of every row
        (role of the reference's batched verify with one graph per key,
        ``crates/model-engine/src/model/trait_impl/verify_e.rs:123``). With recurrent layers the
        graph also holds the step's write-on-accept stash (static buffers, refreshed by every
        replay)."""
        rung = self._rung(len(plan.items))
        key = ("verify", rung, K)
        rows = rung * (K + 1)
        if key not in self.graphs:
            from .batch import SpecStash
            null = self._stage(StepPlan("verify", []), pad_seqs=rung, pad_q=K + 1)
            null.max_ctx, null.max_q_len = self.sched.max_model_len, K + 1
            if self.pool is not None:
                null.spec_stash = SpecStash(null)
            self._forward_select(null, True, False, rows)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            count0 = ops.launch_count
            with _capture(g):
                self._forward_select(null, True, False, rows)
            self.graphs[key] = (g, ops.launch_count - count0, self.last_hidden, null.spec_stash)
        self._stage(plan, pad_seqs=rung, pad_q=K + 1)
        g, launches, hidden, stash = self.graphs[key]
        g.replay()
        ops.launch_count += launches
        self.graph_replays += 1
        self.last_hidden = hidden
        self.pending_stash = stash

    # ------------------------------------------------------------------ pipelined decode
    def can_pipeline(self, plan: StepPlan) -> bool:
        """Plain greedy graph-replayed decode: the only step kind that is launched without waiting."""
        if not (self.graphs_ready() and plan.kind == "decode" and plan.items):
            return False
        if self.decoder.lora is not None and any(i.seq.req.adapter for i in plan.items):
            return False
        if any(i.seq.req.mm is not None for i in plan.items):
            return False
        for it in plan.items:
            p = it.seq.req.params
            if len(it.tokens) != 1 or not it.sample or not p.greedy or p.logprobs or p.needs_host_logits \
                    or p.has_penalties or p.prediction_ids:
                return False
        return True

    def launch_decode(self, plan: StepPlan, ahead: bool = False):
        """Enqueue one decode step (stage, replay, queue the read-back of ids and status) and
        return a handle for ``finish_decode`` without waiting for the device."""
        t0 = time.perf_counter()
        n = len(plan.items)
        if self._decode_graph(plan, True, False, ahead=ahead) is None:
            return None
        par = self._ids_par = self._ids_par ^ 1
        if self._pipe_host is None:
            pin = self.device.type == "cuda"
            self._pipe_host = [torch.zeros(self.max_seqs + 4, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
            self._pipe_ev = [torch.cuda.Event() for _ in range(2)]
        host = self._pipe_host[par]
        host[:n].copy_(self.out_ids[:n], non_blocking=True)
        host[self.max_seqs:self.max_seqs + 4].copy_(ops.runtime(self.device).status, non_blocking=True)
        self._pipe_ev[par].record()
        self.d2h_bytes += 4 * n + 16
        return (plan, par, n, t0)

    def finish_decode(self, handle) -> StepResult:
        plan, par, n, t0 = handle
        self._pipe_ev[par].synchronize()
        host = self._pipe_host[par]
        code = int(host[self.max_seqs])
        if code:
            self.host_status[0] = code
            self.status_pending = True
            self._check_status()
        ids = host[:n].tolist()
        for it in plan.items:
            it.seq.sample_step += 1
        return StepResult([[t] for t in ids], None, hidden=None, device_ms=(time.perf_counter() - t0) * 1e3)

    _ids_par = 0
    _pipe_host = None
    _pipe_ev = None

    # ------------------------------------------------------------------ entry point
    def execute(self, plan: StepPlan) -> StepResult:
        if nvtx.enabled():
            with nvtx.range(f"step:{plan.kind}:{len(plan.items)}"):
                return self._execute(plan)
        return self._execute(plan)

    def _execute(self, plan: StepPlan) -> StepResult:
        dev_cuda = self.device.type == "cuda"
        t0 = time.perf_counter()
        host_logits = any(i.seq.req.params.needs_host_logits or i.seq.req.params.has_penalties
                          for i in plan.items if i.sample)
        want_lp = any(i.seq.req.params.logprobs for i in plan.items)
        greedy = self._set_sampling(plan) if not host_logits else True
        n_sample_rows = sum((i.verify + 1) for i in plan.items if i.sample)
        if n_sample_rows == 0:
            batch = self._stage_with_adapters(plan)
            self.decoder.backbone(batch, self.caches)
            self._after_forward(batch)
            self._post_status()                       # read at the next synchronisation point
            return StepResult([[] for _ in plan.items], device_ms=(time.perf_counter() - t0) * 1e3)
        if host_logits:
            return self._execute_host_logits(plan, t0)
        is_plain_decode = plan.kind == "decode" and all(len(i.tokens) == 1 for i in plan.items)
        uses_adapter = (self.decoder.lora is not None and any(i.seq.req.adapter for i in plan.items)) \
            or any(i.seq.req.mm is not None for i in plan.items)          # rows with their own rotary rows run eagerly too
        K = plan.items[0].verify if plan.items else 0
        uniform_verify = (plan.kind == "verify" and K > 0 and greedy and not want_lp
                          and all(i.verify == K and len(i.tokens) == K + 1 and i.sample for i in plan.items)
                          and self._rung(len(plan.items)) * (K + 1) <= self.stage.max_tokens)
        if is_plain_decode and self.graphs_ready() and not uses_adapter:
            self._decode_graph(plan, greedy, want_lp)
        elif uniform_verify and self.graphs_ready() and not uses_adapter:
            self._verify_graph(plan, K)
        else:
            batch = self._stage_with_adapters(plan)     # steps with adapter rows run eagerly
            self._forward_select(batch, greedy, want_lp, n_sample_rows)
        self.host_ids[:n_sample_rows].copy_(self.out_ids[:n_sample_rows], non_blocking=True)
        if want_lp or not greedy:
            self.host_lp[:n_sample_rows].copy_(self.out_lp[:n_sample_rows], non_blocking=True)
            self.d2h_bytes += 4 * n_sample_rows
        self.d2h_bytes += 4 * n_sample_rows
        self._post_status()
        if dev_cuda:
            torch.cuda.current_stream(self.device).synchronize()
        self._check_status()
        ids = self.host_ids[:n_sample_rows].tolist()
        lps = self.host_lp[:n_sample_rows].tolist() if (want_lp or not greedy) else None
        toks, lpo, r = [], [], 0
        for it in plan.items:
            if not it.sample:
                toks.append([]); lpo.append([])
                continue
            k = it.verify + 1
            toks.append(ids[r:r + k])
            lpo.append(lps[r:r + k] if lps else [])
            it.seq.sample_step += 1
            r += k
        return StepResult(toks, lpo if lps else None, hidden=self.last_hidden,
                          device_ms=(time.perf_counter() - t0) * 1e3)

    def _execute_host_logits(self, plan: StepPlan, t0: float) -> StepResult:
        """Full-logits path: penalties, logit bias, grammar masks, top-n-sigma, top log-probs."""
        from ..sampling.host import sample_rows
        batch = self._stage_with_adapters(plan)
        logits, hidden = self.decoder.forward(batch, self.caches, out_f32=True)
        self._after_forward(batch)
        self.last_hidden = hidden
        self._post_status()
        toks, lps = sample_rows(self, plan, logits)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        self._check_status()
        self.d2h_bytes += logits.numel() * 4
        return StepResult(toks, lps, hidden=hidden, device_ms=(time.perf_counter() - t0) * 1e3)

    # ------------------------------------------------------------------ MTP drafting
    def enable_dflash(self, dc, weights=None, seed: int = 1) -> None:
        """Attach a block drafter (speculative/dflash.py): from now on every target forward also
        writes the drafter's context K/V, and `propose` drafts with it."""
        from ..speculative.dflash import DflashDrafter
        assert not self.graphs, "attach the drafter before the first decode graph is captured"
        self.dflash = DflashDrafter(self, dc, weights, seed)
        self.decoder.side_head = self.dflash

    def propose(self, plan: StepPlan, result: StepResult, accepted: List[int], k: int) -> List[List[int]]:
        """Draft k tokens per sequence with the MTP head, autoregressively: step j feeds the
        previous token and the previous hidden state (target hidden for j = 0)."""
        if k <= 0 or (self.w.mtp is None and self.dflash is None):
            return [[] for _ in plan.items]
        if self.dflash is not None:
            live = [(i, it.seq) for i, it in enumerate(plan.items)
                    if it.sample and accepted[i] > 0 and not it.seq.is_finished()]
            out = [[] for _ in plan.items]
            if live:
                for (i, _), d in zip(live, self.dflash.propose([s for _, s in live], k)):
                    out[i] = d
            self.tp.end_forward()
            return out
        from ..speculative.mtp import mtp_propose
        return mtp_propose(self, plan, result, accepted, k)

    def propose_graphed(self, seqs, first_tok: List[int], hid_rows: List[int], hidden_all: torch.Tensor,
                        k: int) -> Optional[List[List[int]]]:
        """All k draft steps of the MTP head for every sequence as ONE CUDA-graph replay per
        (batch rung, k): one metadata upload (first token, position, block table, hidden row of
        each sequence), one gather of the target hidden rows, the graph, one read-back of
        [rung, k] token ids. Inside the graph, step j derives its positions, KV slots and context
        lengths from step 0's on the device, and feeds its own argmax and hidden state to step
        j + 1 (role of the reference's drafter graphs, one per key,
        ``crates/server/src/scheduler/mtp_step.rs``). Returns None when some sequence has no
        KV block for its last draft position (the caller then drafts step by step)."""
        bs, n = self.block_size, len(seqs)
        for s in seqs:
            if (len(s.tokens) - 1 + k - 1) // bs >= len(s.blocks):
                return None
        rung = self._rung(n)
        S, mb, H, dev = self.sched.max_num_seqs, self.max_blocks, self.cfg.hidden_size, self.device
        if getattr(self, "_mtp_stage", None) is None:
            tot = 4 * S + S * mb
            host = torch.zeros(tot, dtype=torch.int32, pin_memory=True)
            self._mtp_stage = dict(host=host, np=host.numpy(), dev=torch.zeros(tot, dtype=torch.int32, device=dev),
                                   hidden=torch.zeros(S, H, dtype=torch.bfloat16, device=dev),
                                   out=torch.zeros(S, 8, dtype=torch.int32, device=dev),
                                   out_host=torch.zeros(S, 8, dtype=torch.int32, pin_memory=True),
                                   ev=torch.cuda.Event())
        st = self._mtp_stage
        assert k <= st["out"].shape[1]
        d = st["dev"]
        tok_d, pos_d, val_d, row_d, bt_d = d[0:S], d[S:2 * S], d[2 * S:3 * S], d[3 * S:4 * S], d[4 * S:].view(S, mb)
        key = ("mtp", rung, k)
        if key not in self.graphs:
            ar32 = torch.arange(rung, dtype=torch.int32, device=dev)
            ar64 = torch.arange(rung, dtype=torch.int64, device=dev)
            ones = torch.ones(rung, dtype=torch.int32, device=dev)
            zeros = torch.zeros(rung, dtype=torch.int32, device=dev)

            def body():
                toks, hid = tok_d[:rung], st["hidden"][:rung]
                valid = val_d[:rung] > 0
                for j in range(k):
                    pos = pos_d[:rung] + j
                    blk = bt_d[:rung].gather(1, (pos // bs).long()[:, None]).squeeze(1).long()
                    slot = torch.where(valid, blk * bs + (pos % bs).long(), torch.full_like(blk, -1))
                    b = ForwardBatch(token_ids=toks, positions=pos, slot_mapping=slot, q_start=ar32, q_len=ones,
                                     ctx_len=torch.where(valid, pos + 1, ones), block_table=bt_d[:rung],
                                     logit_rows=ar64, max_q_len=1, max_ctx=self.sched.max_model_len,
                                     state_slots=zeros, num_tokens=rung, num_seqs=rung)
                    logits, hid = self.decoder.mtp_forward(toks, hid, b, self.caches)
                    self.tp.end_forward()
                    toks = ops.argmax(logits)
                    st["out"][:rung, j].copy_(toks)
            d.zero_()                                      # null rows for the warm-up and the capture
            body()
            torch.cuda.synchronize(dev)
            g = torch.cuda.CUDAGraph()
            c0 = ops.launch_count
            with _capture(g):
                body()
            self.graphs[key] = (g, ops.launch_count - c0, None, None)
        st["ev"].synchronize()
        a = st["np"]
        a[0:rung], a[S:S + rung], a[2 * S:2 * S + rung], a[3 * S:3 * S + rung] = 0, 0, 0, 0
        a[0:n] = first_tok
        a[S:S + n] = [len(s.tokens) - 1 for s in seqs]
        a[2 * S:2 * S + n] = 1
        a[3 * S:3 * S + n] = hid_rows
        bt = a[4 * S:].reshape(S, mb)
        for i, s in enumerate(seqs):
            bt[i, :len(s.blocks)] = s.blocks
        used = 4 * S + rung * mb
        d[:used].copy_(st["host"][:used], non_blocking=True)
        st["ev"].record()
        torch.index_select(hidden_all, 0, row_d[:n].long(), out=st["hidden"][:n])
        g, launches, _, _ = self.graphs[key]
        g.replay()
        ops.launch_count += launches + 1
        self.graph_replays += 1
        st["out_host"][:rung].copy_(st["out"][:rung], non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        return st["out_host"][:n, :k].tolist()

    # ------------------------------------------------------------------ helpers
    def kv_bytes(self) -> int:
        return self.kv.bytes() + (self.mtp_kv.bytes() if self.mtp_kv else 0)


def plan_kv_blocks(cfg: ModelConfig, w: ModelW, device, block_size: int, utilization: float = 0.9,
                   reserve_bytes: int = 6 << 30, max_blocks: Optional[int] = None) -> int:
    """KV budget: what is left of `utilization` x device memory after the weights and a
    reserve for activations / workspaces / graphs (role of factory/build.rs KV sizing)."""
    dev = torch.device(device)
    kc = kv_config(cfg, w, block_size)
    per_block = kc.block_bytes()
    if w.mtp is not None:
        per_block += kv_config(cfg, w, block_size, mtp=True).block_bytes()
    if dev.type != "cuda":
        return max_blocks or 512
    free, total = torch.cuda.mem_get_info(dev)
    budget = min(free, int(total * utilization) - (total - free)) - reserve_bytes
    n = max(16, budget // max(1, per_block))
    return min(n, max_blocks) if max_blocks else n
