"""The decoder graph: one class assembles every served architecture from per-layer blocks
(attention | gated-delta-net | Mamba2 | MLA mixer, then dense | MoE | no FFN), following the
op order of the reference's circuits (``kernels/circuits/dense_gqa.toml:65-212``,
``blocks/qwen3_hybrid.toml``, ``qwen3_6_moe.toml``, ``nemotron_h.toml``).

The residual stream `x` is bf16 ``[T, hidden]``. Every sub-block is
``x = x + proj(mixer(norm(x)))`` with the residual add fused into the projection GEMM's
epilogue and the norm fused with the activation quantiser of the GEMM that consumes it, so a
dense layer is ten launches. The same code runs on CPU tensors (fp32 restatement of each op:
the oracle) and on CUDA tensors (sm_100a kernels).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from .. import ops
from ..config.model_config import ModelConfig
from ..engine.batch import ForwardBatch
from ..ops import ACT_FOR_WEIGHT, Act
from ..ops import reference as ref
from ..weights.loader import AttnW, FfnW, LayerW, ModelW


class LayerCaches:
    """Per-layer handles into the paged KV cache and the recurrent-state pool."""

    def __init__(self, cfg: ModelConfig, kv=None, state=None, mtp_kv=None):
        self.kv, self.state, self.mtp_kv = kv, state, mtp_kv
        self.kv_index, self.state_index = {}, {}
        a = s = 0
        for i, t in enumerate(cfg.layer_types):
            if t in ("attention", "mla"):
                self.kv_index[i] = a
                a += 1
            else:
                self.state_index[i] = s
                s += 1


class TpContext:
    """How partial sums are combined across tensor-parallel ranks. The single-rank context
    is a no-op (role of the reference's ``SingleGpuBackend``)."""
    size = 1
    rank = 0

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def all_gather_last(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def linear_reduce(self, act: Act, w, residual=None, defer: bool = False):
        """Row-parallel projection + sum over ranks + residual. `defer`: the caller's next step
        is a norm that can perform the sum itself (see parallel.tp.NcclTpContext)."""
        return ops.linear(act, w, residual=residual)

    def sum_deferred(self, y: torch.Tensor, residual=None):
        return y if residual is None else (residual.float() + y.float()).to(torch.bfloat16)

    def end_forward(self) -> None:
        pass


class Decoder:
    def __init__(self, cfg: ModelConfig, weights: ModelW, tp: Optional[TpContext] = None, device=None):
        self.cfg, self.w, self.tp = cfg, weights, tp or TpContext()
        if device is None:                 # tables live where the weights live
            device = weights.embed.device if getattr(weights, "embed", None) is not None else "cpu"
        self.device = torch.device(device)
        rot = cfg.rotary_dim
        self.cos = self.sin = None
        if rot > 0:
            self.cos, self.sin = ref.rope_tables(cfg.max_position, rot, cfg.rope_theta, device=self.device,
                                                 scaling=cfg.rope_scaling)
            if cfg.rope_identity:          # position-free attention in a rotary layout: cos = 1, sin = 0
                self.cos, self.sin = torch.ones_like(self.cos), torch.zeros_like(self.sin)
        self.cos_local = self.sin_local = None
        if rot > 0 and cfg.rope_local_theta > 0:          # windowed layers rotate with their own, unscaled base
            self.cos_local, self.sin_local = ref.rope_tables(cfg.max_position, rot, cfg.rope_local_theta, device=self.device)
        self.scale = cfg.attn_scale if cfg.attn_scale > 0 else 1.0 / math.sqrt(cfg.head_dim)
        self.kv_cal = None                 # cache.fp8_calibration.Fp8KvCalibration while FP8 KV scales are being calibrated
        self.lora = None                   # lora.LoraManager when adapters are served
        self.calib = None                  # dict while calibrating static activation scales (engine/runner.py)
        self.side_head = None              # speculative.dflash.DflashDrafter: sees chosen layers' hidden states of every forward

    # ------------------------------------------------------------------ helpers
    def _norm_act(self, x, w, fmt: str, also_bf16: bool = False, res_only: bool = False) -> Act:
        """RMSNorm(x) encoded for the GEMM that consumes it. When x is a pending cross-rank sum
        the norm kernel performs the sum (+ residual) itself; afterwards ``self.res(x)`` is the
        summed stream. `res_only`: the caller uses that stream only as the residual of the next
        row-parallel projection, so each rank may keep just its own row share."""
        if hasattr(x, "resolve"):
            if w is None:
                x = x.resolve()
            else:
                return x.owner.reduce_norm(x, w, fmt, plus_one=self.cfg.norm_plus_one, eps=self.cfg.rms_eps,
                                           also_bf16=also_bf16, gather_residual=not res_only)
        if w is None:                      # post-norm-only models: the block reads the stream as it is
            a = self._as_act(x if x.dtype == torch.bfloat16 or not x.is_cuda else x.to(torch.bfloat16), fmt)
            if also_bf16 and getattr(a, "bf16", None) is None:
                a.bf16 = x
            return a
        return ops.row_op(x, fmt, ops.IN_RMSNORM, w=w, plus_one=self.cfg.norm_plus_one,
                          eps=self.cfg.rms_eps, also_bf16=also_bf16)[0]

    @staticmethod
    def res(x):
        """The residual-stream tensor behind x (x itself, or the value of a reduced PendingSum)."""
        if hasattr(x, "resolve"):
            return x.value if x.value is not None else x.resolve()
        return x

    @staticmethod
    def full(x):
        """x as a tensor that is complete on every rank."""
        return x.resolve() if hasattr(x, "resolve") else x

    def _add_normed(self, x: torch.Tensor, y: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """x + RMSNorm(y): the sandwich norm of the Gemma family (the block's output is normalised
        before it joins the residual stream)."""
        if not hasattr(y, "resolve") and y.dtype != x.dtype:
            y = y.to(x.dtype)
        n = self._norm_act(y, w, "bf16").data
        return x + n.to(x.dtype)

    @staticmethod
    def _as_act(t: torch.Tensor, fmt: str) -> Act:
        if fmt == "bf16" and t.is_cuda:
            return Act("bf16", t.shape[0], t.shape[1], t, bf16=t)
        return ops.quantize_act(t, fmt)

    # ------------------------------------------------------------------ blocks
    def _lora_for(self, batch: ForwardBatch, li: int):
        if self.lora is None or li < 0 or getattr(batch, "adapter_rows", None) is None:
            return None
        return self.lora

    def attention_block(self, x, lw: LayerW, batch: ForwardBatch, kc, vc, ks, vs, li: int = -1,
                        add_residual: bool = True, kv_layer: int = -1):
        c, w = self.cfg, lw.mixer
        D = c.head_dim
        window = c.window_layers[li] if (c.window_layers and 0 <= li < len(c.window_layers)) else c.sliding_window
        local = window > 0 and self.cos_local is not None
        cos, sin = (self.cos_local, self.sin_local) if local else (self.cos, self.sin)
        rope_pos = batch.positions
        if getattr(batch, "rope_tables", None) is not None:
            # multimodal batch: every row brings its own rotary row (three-axis positions gathered per
            # frequency section), addressed by the row's index
            if local:
                raise NotImplementedError("multimodal rotary positions with per-layer local rotary bases")
            cos, sin = batch.rope_tables
            rope_pos = batch.rope_rows
        lora = self._lora_for(batch, li)
        a = self._norm_act(x, lw.ln1, ACT_FOR_WEIGHT[w.qkv.fmt], also_bf16=lora is not None, res_only=add_residual)
        x = self.res(x)
        res = x if add_residual else None
        defer = add_residual and lora is None
        qkv = ops.linear(a, w.qkv)
        if w.qkv_bias is not None:
            qkv.add_(w.qkv_bias)
        qhs = 2 * D if c.attn_output_gate else D
        if lora is not None:
            # adapter deltas go straight into the fused q|k|v output, before norm / rope / cache write
            xb = a.bf16 if getattr(a, "bf16", None) is not None else a.data
            if not c.attn_output_gate:
                lora.apply(qkv, xb, li, "q", batch.adapter_rows, 0)
            lora.apply(qkv, xb, li, "k", batch.adapter_rows, w.heads * qhs)
            lora.apply(qkv, xb, li, "v", batch.adapter_rows, w.heads * qhs + w.kv_heads * D)
        qn, kn = w.q_norm, w.k_norm
        if c.qk_norm_full and qn is not None:
            # the norm spans the whole projection (all heads): normalised in place here, then the
            # fused kernel only rotates and writes the cache
            nq, nk = w.heads * qhs, w.kv_heads * D
            for lo, n, wt in ((0, nq, qn), (nq, nk, kn)):
                part = qkv[:, lo:lo + n].float()
                part = part * torch.rsqrt(part.pow(2).mean(-1, keepdim=True) + c.rms_eps) * wt.float()
                qkv[:, lo:lo + n] = part.to(qkv.dtype)
            qn = kn = None
        q = ops.qk_norm_rope_kvwrite(
            qkv, Hq=w.heads, Hkv=w.kv_heads, D=D, positions=rope_pos, slots=batch.slot_mapping,
            k_cache=kc, v_cache=vc, q_norm_w=qn, k_norm_w=kn, plus_one=c.norm_plus_one,
            eps=c.rms_eps, cos=cos, sin=sin, q_head_stride=qhs, k_scale=ks, v_scale=vs,
            amax=self.kv_cal.amax_for(kv_layer) if (self.kv_cal is not None and kv_layer >= 0) else None)
        fmt = ACT_FOR_WEIGHT[w.o.fmt]
        static = w.o_in_scale if (fmt == "nvfp4" and self.calib is None and not c.attn_output_gate) else 0.0
        if static > 0.0 and lora is None:
            # the attention kernel's final store quantises for o_proj with the calibrated scale
            oa = ops.paged_attention(q, kc, vc, batch.block_table, batch.q_start, batch.q_len, batch.ctx_len,
                                     max_q_len=batch.max_q_len, max_ctx=batch.max_ctx, scale=self.scale,
                                     k_scale=ks, v_scale=vs, window=window, quant_out=static)
            return self.tp.linear_reduce(oa, w.o, residual=res, defer=defer)
        o = ops.paged_attention(q, kc, vc, batch.block_table, batch.q_start, batch.q_len, batch.ctx_len,
                                max_q_len=batch.max_q_len, max_ctx=batch.max_ctx, scale=self.scale,
                                k_scale=ks, v_scale=vs, window=window)
        o = o.view(o.shape[0], w.heads * D)
        if self.calib is not None:
            m = o.float().abs().max()
            self.calib[id(w)] = torch.maximum(self.calib[id(w)], m) if id(w) in self.calib else m
        if c.attn_output_gate:
            oa = ops.row_op(o, fmt, ops.IN_SIGMOID_GATE, gate=qkv, head_dim=D, gate_head_stride=2 * D,
                            gate_head_off=D)[0]
        else:
            oa = ops.quantize_act(o, fmt, static_scale=static) if fmt == "nvfp4" else self._as_act(o, fmt)
        y = self.tp.linear_reduce(oa, w.o, residual=res, defer=defer)
        if lora is not None and not c.attn_output_gate:
            lora.apply(y, o, li, "o", batch.adapter_rows)
        return y

    def dense_ffn(self, a: Act, w: FfnW, residual, lora=None, li: int = -1, rows=None) -> torch.Tensor:
        c = self.cfg
        fmt_d = ACT_FOR_WEIGHT[w.down.fmt]
        hb = None
        if c.ffn_act == "relu2":
            up = ops.linear(a, w.gate_up)
            h = ops.row_op(up, fmt_d, ops.IN_RELU2, also_bf16=lora is not None)[0]
        elif c.ffn_act == "geglu":
            gu = ops.linear(a, w.gate_up)                     # gate | up halves
            inter = gu.shape[1] // 2
            hb = (torch.nn.functional.gelu(gu[:, :inter].float(), approximate="tanh") * gu[:, inter:].float()
                  ).to(torch.bfloat16)
            h = self._as_act(hb, fmt_d)
        elif w.interleaved:
            static = w.down_in_scale if (fmt_d == "nvfp4" and self.calib is None) else 0.0
            if static > 0.0 and lora is None:
                # SwiGLU output quantised inside the GEMM epilogue with the calibrated scale
                h = ops.linear(a, w.gate_up, swiglu=True, quant_out=static)
            else:
                hb = ops.linear(a, w.gate_up, swiglu=True)
                if self.calib is not None:
                    m = hb.float().abs().max()
                    self.calib[id(w)] = torch.maximum(self.calib[id(w)], m) if id(w) in self.calib else m
                h = ops.quantize_act(hb, fmt_d, static_scale=static) if fmt_d == "nvfp4" else self._as_act(hb, fmt_d)
        else:
            gu = ops.linear(a, w.gate_up)
            static = w.down_in_scale if (fmt_d == "nvfp4" and self.calib is None) else 0.0
            h = ops.row_op(gu, fmt_d, ops.IN_SILU_MUL, also_bf16=lora is not None, static_scale=static)[0]
        y = self.tp.linear_reduce(h, w.down, residual=residual, defer=residual is not None and lora is None)
        if lora is not None:
            if hb is None:
                hb = h.bf16 if getattr(h, "bf16", None) is not None else h.data
            lora.apply(y, hb, li, "down", rows)
        return y

    def ffn_block(self, x, lw: LayerW, batch: Optional[ForwardBatch] = None, li: int = -1):
        if lw.ffn_kind == "none":
            return x
        if lw.ffn_kind == "dense":
            plain = lw.post_ffn is None and self.cfg.residual_multiplier == 1.0
            a = self._norm_act(x, lw.ln2, ACT_FOR_WEIGHT[lw.ffn.gate_up.fmt], res_only=plain)
            x = self.res(x)
            lora = self._lora_for(batch, li) if batch is not None else None
            rows = batch.adapter_rows if lora is not None else None
            if lw.post_ffn is not None:
                y = self.dense_ffn(a, lw.ffn, None, lora, li, rows)
                return self._add_normed(x, y, lw.post_ffn)
            if self.cfg.residual_multiplier != 1.0:
                y = self.dense_ffn(a, lw.ffn, None, lora, li, rows)
                return x + (self.full(y).float() * self.cfg.residual_multiplier).to(x.dtype)
            return self.dense_ffn(a, lw.ffn, x, lora, li, rows)
        from .moe import moe_block
        return moe_block(self, x, lw)

    def layer(self, i: int, x, lw: LayerW, batch: ForwardBatch, caches: LayerCaches, kv=None, kv_idx=None):
        if lw.kind == "attention":
            kv = kv or caches.kv
            j = caches.kv_index[i] if kv_idx is None else kv_idx
            if lw.post_attn is not None or self.cfg.residual_multiplier != 1.0:
                x = self.full(x)
            if lw.post_attn is not None:
                y = self.attention_block(x, lw, batch, kv.k[j], kv.v[j], kv.k_scale[j], kv.v_scale[j], li=i,
                                         add_residual=False, kv_layer=j if kv is caches.kv else -1)
                x = self._add_normed(x, y, lw.post_attn)
            elif self.cfg.residual_multiplier != 1.0:
                y = self.attention_block(x, lw, batch, kv.k[j], kv.v[j], kv.k_scale[j], kv.v_scale[j], li=i,
                                         add_residual=False, kv_layer=j if kv is caches.kv else -1)
                x = x + (self.full(y).float() * self.cfg.residual_multiplier).to(x.dtype)
            else:
                x = self.attention_block(x, lw, batch, kv.k[j], kv.v[j], kv.k_scale[j], kv.v_scale[j], li=i,
                                         kv_layer=j if kv is caches.kv else -1)
        elif lw.kind == "gdn":
            from .recurrent import gdn_block
            x = gdn_block(self, x, lw, batch, caches.state, caches.state_index[i])
        elif lw.kind == "kda":
            from .recurrent import kda_block
            x = kda_block(self, x, lw, batch, caches.state, caches.state_index[i])
        elif lw.kind == "mamba2":
            from .recurrent import mamba2_block
            x = mamba2_block(self, x, lw, batch, caches.state, caches.state_index[i])
        elif lw.kind == "mla":
            from .mla import mla_block
            kv = kv or caches.kv
            j = caches.kv_index[i] if kv_idx is None else kv_idx
            x = mla_block(self, x, lw, batch, kv, j)
        return self.ffn_block(x, lw, batch, i)

    # ------------------------------------------------------------------ full forward
    def embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        x = ops.embed(token_ids, self.w.embed)
        if self.cfg.embed_scale != 1.0:
            x = x * torch.tensor(self.cfg.embed_scale, dtype=torch.bfloat16).to(x.dtype)
        return x

    def backbone(self, batch: ForwardBatch, caches: LayerCaches) -> torch.Tensor:
        """Token ids -> final residual stream [T, hidden] (before the final norm)."""
        x = self.embed(batch.token_ids)
        if getattr(batch, "embed_override", None) is not None:
            rows, emb = batch.embed_override
            x = x.index_copy(0, rows, emb.to(x.dtype))
        side = self.side_head
        if side is not None:
            side.begin(x.shape[0])
        if self.cfg.hc_mult > 1:
            return self._backbone_highway(x, batch, caches)
        for i, lw in enumerate(self.w.layers):
            x = self.layer(i, x, lw, batch, caches)
            if side is not None and i in side.capture_ids:
                x = self.full(x)
                side.capture(i, x)
        if side is not None:
            side.absorb(batch)
        return x

    def _backbone_highway(self, x, batch: ForwardBatch, caches: LayerCaches) -> torch.Tensor:
        """Hyper-connection models: the residual stream is hc fp32 copies per token. Each block reads a
        learned mixture of the copies (``hc_pre``: one fused kernel for the statistics, the mixing
        projection, the gates and the Sinkhorn-normalised combination matrix) and its output is
        written back into every copy (``hc_post``); the final norm sees the mean of the copies.
        Dense GQA blocks only (the block output is taken without its residual add). Reference:
        kernels/gb10/common/glm5next_mhc.cu, deepseek-v4-flash/nvfp4/hyper_connection.cu."""
        from ..ops import highway as hw
        c = self.cfg
        if self.tp.size > 1:
            raise NotImplementedError("hyper-connections are served on one rank")
        kw = dict(norm_eps=c.rms_eps, hc_eps=c.hc_eps, iters=c.hc_sinkhorn_iters)
        streams = hw.hc_expand(x, c.hc_mult)
        for i, lw in enumerate(self.w.layers):
            if lw.kind != "attention" or lw.ffn_kind != "dense":
                raise NotImplementedError("hyper-connections: attention + dense feed-forward layers only")
            kv, j = caches.kv, caches.kv_index[i]
            y, post, comb = hw.hc_pre(streams, *lw.hc_attn, **kw)
            f = self.attention_block(y, lw, batch, kv.k[j], kv.v[j], kv.k_scale[j], kv.v_scale[j], li=i,
                                     add_residual=False, kv_layer=j)
            streams = hw.hc_post(self.full(f), streams, post, comb)
            y, post, comb = hw.hc_pre(streams, *lw.hc_ffn, **kw)
            a = self._norm_act(y, lw.ln2, ACT_FOR_WEIGHT[lw.ffn.gate_up.fmt])
            f = self.dense_ffn(a, lw.ffn, None, None, i, None)
            streams = hw.hc_post(self.full(f), streams, post, comb)
        return hw.hc_head_mean(streams)

    def logits(self, hidden_rows, final_norm=None, out_f32: bool = False, gather: bool = True) -> torch.Tensor:
        """Final norm + (vocab-parallel) lm_head on the selected rows."""
        a = self._norm_act(hidden_rows, self.w.final_norm if final_norm is None else final_norm, "bf16")
        lg = ops.linear(a, self.w.lm_head, out_f32=out_f32)
        if self.cfg.logits_divisor != 1.0:
            lg = (lg.float() / self.cfg.logits_divisor).to(lg.dtype)
        cap = self.cfg.final_logit_softcap
        if cap > 0:
            lg = (torch.tanh(lg.float() / cap) * cap).to(lg.dtype)
        return self.tp.all_gather_last(lg) if gather else lg

    def forward(self, batch: ForwardBatch, caches: LayerCaches, out_f32: bool = False,
                gather_logits: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (logits [R, vocab], hidden [R, hidden]) for batch.logit_rows. With
        `gather_logits` off a tensor-parallel rank returns its own vocabulary shard
        [R, vocab / size] (greedy selection then merges per-rank maxima instead)."""
        x = self.backbone(batch, caches)
        if batch.logit_rows.numel() != x.shape[0]:
            rows = self.full(x).index_select(0, batch.logit_rows)
        else:
            rows = x
        lg = self.logits(rows, out_f32=out_f32, gather=gather_logits)
        return lg, self.res(rows)

    # ------------------------------------------------------------------ MTP draft head
    def mtp_forward(self, token_ids, hidden, batch: ForwardBatch, caches: LayerCaches) -> Tuple[torch.Tensor, torch.Tensor]:
        """One multi-token-prediction step: embed(next token) || target hidden -> two norms ->
        concat -> fc -> one decoder layer over the head's own KV cache -> norm -> lm_head
        (kernels/circuits/blocks/qwen3_hybrid.toml:285-340). Returns (logits, hidden)."""
        m, c = self.w.mtp, self.cfg
        e = self._norm_act(self.embed(token_ids), m.norm_emb, "bf16").bf16
        h = self._norm_act(hidden, m.norm_hid, "bf16").bf16
        cat = torch.cat([e, h], dim=-1).contiguous()
        x = ops.linear(self._as_act(cat, "bf16"), m.fc)
        x = self.layer(c.num_layers, x, m.layer, batch, caches, kv=caches.mtp_kv, kv_idx=0)
        rows = self.full(x).index_select(0, batch.logit_rows) if batch.logit_rows.numel() != x.shape[0] else x
        lg = self.logits(rows, final_norm=m.final_norm)
        return lg, self.res(rows)
