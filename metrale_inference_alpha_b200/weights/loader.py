"""HF tensor names -> typed, fused, sharded serving weights.

``read_linear`` recognises the checkpoint dialects (ModelOpt NVFP4 ``.weight/.weight_scale/
.weight_scale_2``, compressed-tensors NVFP4 ``.weight_packed/.weight_scale/
.weight_global_scale`` with the global scale inverted at load, FP8 block-scaled
``.weight_scale_inv`` or 2-D ``.weight_scale``, FP8 per-row ``.weight_scale`` of N elements,
a scalar ``.weight_scale`` replicated over the block grid, raw bf16 with optional runtime
quantisation). Tensor-parallel sharding follows the usual scheme: column-parallel q/k/v/gate/up
(whole heads per rank), row-parallel o/down, replicated norms and routers, experts split by
index for expert parallelism.
Role of the reference's ``crates/model-layers/src/quant_format/``, ``weight_map/`` and
``crates/model-arch/src/tp_shard.rs`` (+ ``tp_shard/quant_shard.rs``, ``tp_shard/gdn.rs``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.model_config import ModelConfig
from ..ops import QuantWeight
from .source import SyntheticSource, TensorSource


# ----------------------------------------------------------------------------- linear readers
def read_linear(src: TensorSource, prefix: str, device, runtime_fmt: Optional[str] = None) -> QuantWeight:
    """Read one linear layer in whatever dialect the checkpoint uses. A raw bf16 tensor is
    quantised to `runtime_fmt` when that is given (the "Bf16Raw" path)."""
    has = src.has
    dev = torch.device(device)
    if has(f"{prefix}.weight_packed"):                       # compressed-tensors NVFP4
        q = src.get(f"{prefix}.weight_packed").to(dev)
        sf = src.get(f"{prefix}.weight_scale").to(dev)
        g = 1.0 / float(src.get(f"{prefix}.weight_global_scale").float().reshape(-1)[0])
        return _nvfp4(q, sf, g)
    w = src.get(f"{prefix}.weight").to(dev)
    if w.dtype == torch.float8_e4m3fn:
        w = w.view(torch.uint8)
    if has(f"{prefix}.weight_scale_2"):                      # ModelOpt NVFP4
        sf = src.get(f"{prefix}.weight_scale").to(dev)
        g = float(src.get(f"{prefix}.weight_scale_2").float().reshape(-1)[0])
        return _nvfp4(w, sf, g)
    if w.dtype == torch.uint8:
        N, K = w.shape
        if has(f"{prefix}.weight_scale_inv"):
            s = src.get(f"{prefix}.weight_scale_inv").to(dev).float()
        else:
            s = src.get(f"{prefix}.weight_scale").to(dev).float()
        if s.numel() == N and not (s.ndim == 2 and s.shape == ((N + 127) // 128, (K + 127) // 128)):
            return QuantWeight("fp8_row", N, K, w.contiguous(), s.reshape(N).contiguous())
        if s.numel() == 1:                                   # per-tensor scale -> block grid
            s = s.reshape(1, 1).expand((N + 127) // 128, (K + 127) // 128)
        return QuantWeight("fp8_block", N, K, w.contiguous(), s.contiguous())
    if runtime_fmt and runtime_fmt != "bf16":
        return ops.make_weight(w.float(), runtime_fmt).to(dev) if dev.type == "cuda" else ops.make_weight(w.float(), runtime_fmt)
    return QuantWeight("bf16", w.shape[0], w.shape[1], w.to(torch.bfloat16).contiguous())


def _nvfp4(q, sf, g) -> QuantWeight:
    if sf.dtype == torch.float8_e4m3fn:
        sf = sf.view(torch.uint8)
    return QuantWeight("nvfp4", q.shape[0], q.shape[1] * 2, q.contiguous(), sf.contiguous(), g)


def slice_rows(w: QuantWeight, lo: int, hi: int) -> QuantWeight:
    out = QuantWeight(w.fmt, hi - lo, w.K, w.data[lo:hi].contiguous(), None, w.gscale)
    if w.fmt in ("fp8_row", "nvfp4"):
        out.scale = w.scale[lo:hi].contiguous()
    elif w.fmt == "fp8_block":
        assert lo % 128 == 0, "row shard must start on a 128-row scale block"
        out.scale = w.scale[lo // 128:(hi + 127) // 128].contiguous()
    if w.row_gscale is not None:
        out.row_gscale = w.row_gscale[lo:hi].contiguous()
    return out


def slice_cols(w: QuantWeight, lo: int, hi: int) -> QuantWeight:
    if w.fmt == "bf16":
        return QuantWeight("bf16", w.N, hi - lo, w.data[:, lo:hi].contiguous())
    if w.fmt == "fp8_row":
        return QuantWeight("fp8_row", w.N, hi - lo, w.data[:, lo:hi].contiguous(), w.scale)
    if w.fmt == "fp8_block":
        assert lo % 128 == 0, "column shard must start on a 128-column scale block"
        return QuantWeight("fp8_block", w.N, hi - lo, w.data[:, lo:hi].contiguous(),
                           w.scale[:, lo // 128:(hi + 127) // 128].contiguous())
    assert lo % 16 == 0 and hi % 16 == 0
    return QuantWeight("nvfp4", w.N, hi - lo, w.data[:, lo // 2:hi // 2].contiguous(),
                       w.scale[:, lo // 16:hi // 16].contiguous(), w.gscale, w.row_gscale)


def finalize(w: QuantWeight) -> QuantWeight:
    if w.data.is_cuda and w.fmt == "nvfp4" and w.sf_tiled is None:
        w.prepare_cuda()
    return w


# ----------------------------------------------------------------------------- typed modules
@dataclass
class AttnW:
    qkv: QuantWeight = None
    o: QuantWeight = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    qkv_bias: Optional[torch.Tensor] = None   # bf16 [q | k | v rows of this rank]
    o_in_scale: float = 0.0   # NVFP4: calibrated global scale of o_proj's input (0 = per-token dynamic)
    heads: int = 0            # local q heads
    kv_heads: int = 0         # local kv heads
    kv_scale: Optional[tuple] = None   # (k_scale, v_scale) dequant multipliers from the checkpoint, or None


@dataclass
class FfnW:
    gate_up: QuantWeight = None      # swiglu: rows interleaved (gate_j, up_j) or gate | up halves; relu2: up only
    down: QuantWeight = None
    interleaved: bool = False        # True -> the GEMM epilogue applies SwiGLU
    down_in_scale: float = 0.0       # NVFP4: calibrated global scale of down's input (0 = per-token dynamic)


@dataclass
class MoeW:
    router: QuantWeight = None
    bias: Optional[torch.Tensor] = None
    experts: List[FfnW] = field(default_factory=list)     # local experts
    expert_lo: int = 0
    shared: Optional[FfnW] = None
    shared_gate: Optional[QuantWeight] = None
    shared_replicated: bool = False                        # expert parallelism keeps the whole shared expert on every rank
    grouped: Optional[object] = None                       # stacked device layout for the grouped GEMM
    router_ext: Optional[QuantWeight] = None               # router rows + the shared expert's gate row (shared expert folded into `grouped`)
    paged: Optional[object] = None                         # storage.expert_store.PagedExperts: the experts live in a store and are paged into an arena
    paged_layer: int = 0                                   # this layer's index in that store


@dataclass
class KdaW:
    in_qkv: QuantWeight = None       # rows q | k | v, heads contiguous
    f_a: QuantWeight = None          # hidden -> rank (decay projection, first half)
    f_b: QuantWeight = None          # rank -> H D
    b_proj: QuantWeight = None       # hidden -> H (beta logits), bf16
    g_a: QuantWeight = None          # hidden -> rank (output gate)
    g_b: QuantWeight = None          # rank -> H D
    conv_w: torch.Tensor = None      # [3 H D, taps] fp32, q | k | v
    A_log: torch.Tensor = None       # [H]
    dt_bias: torch.Tensor = None     # [H D]
    norm_w: torch.Tensor = None      # [D] fp32
    out: QuantWeight = None
    heads: int = 0


@dataclass
class GdnW:
    in_qkvz: QuantWeight = None
    in_ba: QuantWeight = None
    conv_w: torch.Tensor = None      # [C, taps] fp32
    A_log: torch.Tensor = None
    dt_bias: torch.Tensor = None
    norm_w: torch.Tensor = None
    out: QuantWeight = None
    k_heads: int = 0
    v_heads: int = 0


@dataclass
class MambaW:
    in_proj: QuantWeight = None
    conv_w: torch.Tensor = None
    conv_b: Optional[torch.Tensor] = None
    A_log: torch.Tensor = None
    D: torch.Tensor = None
    dt_bias: torch.Tensor = None
    norm_w: torch.Tensor = None
    out: QuantWeight = None
    heads: int = 0
    groups: int = 0


@dataclass
class MlaW:
    q_a: Optional[QuantWeight] = None
    q_a_norm: Optional[torch.Tensor] = None
    q_b: QuantWeight = None
    kv_a: QuantWeight = None
    kv_a_norm: torch.Tensor = None
    w_uk: torch.Tensor = None        # [H, nope, kv_lora] bf16 (absorbed)
    w_uv: torch.Tensor = None        # [H, v, kv_lora] bf16
    o: QuantWeight = None
    heads: int = 0
    # sparse-attention indexer (replicated across tensor-parallel ranks so that every rank selects the same tokens)
    idx_q: Optional[QuantWeight] = None          # query latent (or hidden) -> Hi * Di
    idx_k: Optional[QuantWeight] = None          # hidden -> Di
    idx_k_norm: Optional[torch.Tensor] = None    # LayerNorm weight | bias, fp32 [2, Di]
    idx_w: Optional[QuantWeight] = None          # hidden -> Hi (head weights), bf16


@dataclass
class LayerW:
    kind: str = "attention"
    ffn_kind: str = "dense"
    ln1: torch.Tensor = None
    ln2: Optional[torch.Tensor] = None
    post_attn: Optional[torch.Tensor] = None     # Gemma sandwich norms: applied to the block's output
    post_ffn: Optional[torch.Tensor] = None
    mixer: object = None
    ffn: object = None
    hc_attn: Optional[tuple] = None              # hyper-connection site in front of the mixer: (fn bf16, scale fp32 [3], base fp32)
    hc_ffn: Optional[tuple] = None               # ... and in front of the feed-forward block


@dataclass
class MtpW:
    fc: QuantWeight = None
    norm_emb: torch.Tensor = None
    norm_hid: torch.Tensor = None
    final_norm: torch.Tensor = None
    layer: LayerW = None


@dataclass
class ModelW:
    embed: torch.Tensor = None           # bf16 [V, H]
    lm_head: QuantWeight = None          # bf16, vocab-parallel under TP
    final_norm: torch.Tensor = None
    layers: List[LayerW] = field(default_factory=list)
    mtp: Optional[MtpW] = None
    vocab_lo: int = 0
    vocab_hi: int = 0

    def nbytes(self) -> int:
        n = 0

        def visit(o):
            nonlocal n
            if isinstance(o, QuantWeight):
                n += o.nbytes()
            elif torch.is_tensor(o):
                n += o.numel() * o.element_size()
            elif isinstance(o, (list, tuple)):
                for x in o:
                    visit(x)
            elif hasattr(o, "__dataclass_fields__"):
                for f in o.__dataclass_fields__:
                    visit(getattr(o, f))
        visit(self)
        return n


# ----------------------------------------------------------------------------- module loaders
class Loader:
    def __init__(self, cfg: ModelConfig, src: TensorSource, device="cpu", tp_rank: int = 0, tp_size: int = 1,
                 ep_rank: int = 0, ep_size: int = 1):
        self.cfg, self.src, self.dev = cfg, src, torch.device(device)
        self.tp_rank, self.tp_size, self.ep_rank, self.ep_size = tp_rank, tp_size, ep_rank, ep_size
        self.fmt = cfg.weight_format

    def vec(self, name, dtype=torch.bfloat16):
        return self.src.get(name).to(self.dev).to(dtype).contiguous()

    def lin(self, prefix, quant=True) -> QuantWeight:
        return read_linear(self.src, prefix, self.dev, self.fmt if quant else None)

    def input_scale(self, prefix: str) -> float:
        """Calibrated global scale of an NVFP4 linear's input (ModelOpt's `<linear>.input_scale`,
        amax / (6 * 448)); 0.0 when the checkpoint carries none."""
        name = f"{prefix}.input_scale"
        if self.fmt != "nvfp4" or not self.src.has(name):
            return 0.0
        v = float(self.src.get(name).float().reshape(-1)[0])
        return v if v > 0.0 and v == v and v != float("inf") else 0.0

    def _shard(self, n: int):
        assert n % self.tp_size == 0, f"{n} not divisible by tp {self.tp_size}"
        per = n // self.tp_size
        return self.tp_rank * per, (self.tp_rank + 1) * per

    # ---- attention
    def attention(self, p: str) -> AttnW:
        c = self.cfg
        q, k, v, o = (self.lin(f"{p}.{n}_proj") for n in "qkvo")
        per_q = c.head_dim * (2 if c.attn_output_gate else 1)
        rope_perm_q = rope_perm_k = None
        if c.rope_interleaved and c.rotary_dim > 0:
            # the checkpoint rotates neighbouring pairs (2i, 2i + 1); the kernels rotate (i, i + r/2):
            # re-order the rotary rows of every q / k head (q.k is invariant under a shared permutation)
            r, D = c.rotary_dim, c.head_dim
            head = list(range(0, r, 2)) + list(range(1, r, 2)) + list(range(r, D))
            mk = lambda n: torch.tensor([h * D + j for h in range(n) for j in head], device=q.data.device)
            rope_perm_q, rope_perm_k = mk(c.num_heads), mk(c.num_kv_heads)
            q, k = ops.permute_rows(q, rope_perm_q), ops.permute_rows(k, rope_perm_k)
        hq = c.num_heads // self.tp_size
        if self.tp_size > 1:
            lo, hi = self._shard(c.num_heads)
            q = slice_rows(q, lo * per_q, hi * per_q)
            o = slice_cols(o, lo * c.head_dim, hi * c.head_dim)
            if c.num_kv_heads >= self.tp_size:
                klo, khi = self._shard(c.num_kv_heads)
            else:                                            # replicate kv heads across rank groups
                rep = self.tp_size // c.num_kv_heads
                klo = self.tp_rank // rep
                khi = klo + 1
            k = slice_rows(k, klo * c.head_dim, khi * c.head_dim)
            v = slice_rows(v, klo * c.head_dim, khi * c.head_dim)
            hkv = khi - klo
        else:
            hkv = c.num_kv_heads
        w = AttnW(finalize(ops.concat_weights([q, k, v])), finalize(o), heads=hq, kv_heads=hkv)
        w.o_in_scale = self.input_scale(f"{p}.o_proj")
        if c.attn_bias and self.src.has(f"{p}.q_proj.bias"):
            qb, kb, vb = (self.src.get(f"{p}.{n}_proj.bias").to(self.dev).to(torch.bfloat16) for n in "qkv")
            if rope_perm_q is not None:
                qb, kb = qb[rope_perm_q.to(qb.device)], kb[rope_perm_k.to(kb.device)]
            if self.tp_size > 1:
                qb = qb[lo * per_q:hi * per_q]
                kb, vb = kb[klo * c.head_dim:khi * c.head_dim], vb[klo * c.head_dim:khi * c.head_dim]
            w.qkv_bias = torch.cat([qb, kb, vb]).contiguous()
        if self.src.has(f"{p}.q_norm.weight"):
            w.q_norm, w.k_norm = self.vec(f"{p}.q_norm.weight"), self.vec(f"{p}.k_norm.weight")
            if c.qk_norm_full and self.tp_size > 1:
                raise NotImplementedError("a q / k norm that spans all heads is served on single-rank engines")
        # per-layer FP8 KV scales, in whichever of the three spellings the exporter used
        from .kv_scales import load_kv_scales
        w.kv_scale = load_kv_scales(self.src, {0: p}).get(0)
        return w

    # ---- dense ffn
    def ffn(self, p: str, names=("gate_proj", "up_proj", "down_proj"), shard: bool = True) -> FfnW:
        c = self.cfg
        up = self.lin(f"{p}.{names[1]}")
        down = self.lin(f"{p}.{names[2]}")
        gate = self.lin(f"{p}.{names[0]}") if c.ffn_act in ("swiglu", "geglu") else None
        if shard and self.tp_size > 1:
            lo, hi = self._shard(up.N)
            up, down = slice_rows(up, lo, hi), slice_cols(down, lo, hi)
            if gate is not None:
                gate = slice_rows(gate, lo, hi)
        gs = self.input_scale(f"{p}.{names[2]}")
        if gate is None:
            return FfnW(finalize(up), finalize(down), down_in_scale=gs)
        gu = ops.concat_weights([gate, up])
        if gu.fmt == "fp8_block" or c.ffn_act == "geglu":
            # 128x128 scale blocks forbid a row-interleave, and the GEMM epilogue knows SwiGLU only:
            # keep gate | up halves
            return FfnW(finalize(gu), finalize(down), down_in_scale=gs)
        I = up.N
        perm = torch.stack([torch.arange(I), torch.arange(I) + I], 1).reshape(-1).to(gu.data.device)
        return FfnW(finalize(ops.permute_rows(gu, perm)), finalize(down), interleaved=True, down_in_scale=gs)

    # ---- layers
    def layer(self, p: str, lt: str, ft: str, names=None) -> LayerW:
        from . import loader_ext
        c = self.cfg
        L = LayerW(kind=lt, ffn_kind=ft)
        L.ln1 = self.vec(f"{p}.input_layernorm.weight") if c.pre_norms else None
        if lt == "attention":
            L.mixer = self.attention(f"{p}.self_attn")
        elif lt == "gdn":
            L.mixer = loader_ext.gdn(self, f"{p}.linear_attn")
        elif lt == "mla":
            L.mixer = loader_ext.mla(self, f"{p}.self_attn")
        elif lt == "kda":
            L.mixer = loader_ext.kda(self, f"{p}.self_attn")
        if ft != "none":
            if c.post_norms and c.post_norm_names == "olmo2":     # post-norm only: no norm in front of the blocks
                L.post_attn = self.vec(f"{p}.post_attention_layernorm.weight")
                L.post_ffn = self.vec(f"{p}.post_feedforward_layernorm.weight")
            elif c.post_norms and c.post_norm_names == "glm":
                L.post_attn = self.vec(f"{p}.post_self_attn_layernorm.weight")
                L.ln2 = self.vec(f"{p}.post_attention_layernorm.weight")
                L.post_ffn = self.vec(f"{p}.post_mlp_layernorm.weight")
            elif c.post_norms:        # Gemma: the norm named post_attention acts on the attention output
                L.post_attn = self.vec(f"{p}.post_attention_layernorm.weight")
                L.ln2 = self.vec(f"{p}.pre_feedforward_layernorm.weight")
                L.post_ffn = self.vec(f"{p}.post_feedforward_layernorm.weight")
            else:
                L.ln2 = self.vec(f"{p}.post_attention_layernorm.weight")
        if ft == "dense":
            L.ffn = self.ffn(f"{p}.mlp")
        elif ft == "moe":
            L.ffn = loader_ext.moe(self, f"{p}.mlp")
        if c.hc_mult > 1:
            site = lambda q: (self.src.get(f"{q}.fn").to(self.dev).to(torch.bfloat16).contiguous(),
                              self.vec(f"{q}.scale", torch.float32), self.vec(f"{q}.base", torch.float32))
            L.hc_attn, L.hc_ffn = site(f"{p}.attn_hc"), site(f"{p}.ffn_hc")
        return L

    def load(self) -> ModelW:
        from . import loader_ext
        c = self.cfg
        if c.arch == "nemotron_h":
            return loader_ext.load_nemotron(self)
        m = ModelW()
        m.embed = self.vec("model.embed_tokens.weight")
        m.final_norm = self.vec("model.norm.weight")
        head = QuantWeight("bf16", c.vocab_size, c.hidden_size, m.embed) if c.tie_embeddings else self.lin("lm_head", quant=False)
        m.vocab_lo, m.vocab_hi = 0, c.vocab_size
        if self.tp_size > 1:
            per = (c.vocab_size + self.tp_size - 1) // self.tp_size
            m.vocab_lo, m.vocab_hi = self.tp_rank * per, min(c.vocab_size, (self.tp_rank + 1) * per)
            head = slice_rows(head, m.vocab_lo, m.vocab_hi)
        m.lm_head = head
        for i in range(c.num_layers):
            m.layers.append(self.layer(f"model.layers.{i}", c.layer_types[i], c.ffn_types[i]))
        if c.mtp_layers:
            mt = MtpW()
            mt.fc = self.lin("mtp.fc", quant=False)
            mt.norm_emb = self.vec("mtp.pre_fc_norm_embedding.weight")
            mt.norm_hid = self.vec("mtp.pre_fc_norm_hidden.weight")
            mt.final_norm = self.vec("mtp.norm.weight")
            lt = "mla" if c.arch == "deepseek_mla" else "attention"
            mt.layer = self.layer("mtp.layers.0", lt, "moe" if c.num_experts else "dense")
            m.mtp = mt
        return m


def load_weights(cfg: ModelConfig, src: Optional[TensorSource] = None, device="cpu", tp_rank=0, tp_size=1,
                 ep_rank=0, ep_size=1, seed: int = 0) -> ModelW:
    """Load (or synthesise, when `src` is None) the serving weights of `cfg` for this rank."""
    if src is None:
        src = SyntheticSource(cfg, seed=seed, device=device)
    return Loader(cfg, src, device, tp_rank, tp_size, ep_rank, ep_size).load()
