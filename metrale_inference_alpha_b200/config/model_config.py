"""Model shape + precision description, parsed from a HF ``config.json`` or built from a preset.

Covers the architectures the engine serves: dense GQA decoders (Llama / Qwen3 style),
hybrid gated-delta-net + gated-attention MoE (Qwen3.5 / 3.6 style), Nemotron-H hybrids
(Mamba2 + attention + squared-ReLU MLP / MoE) and DeepSeek-V3 style MLA MoE.
Role of the reference's ``crates/config`` (``ModelConfig`` and the per-family parsers in
``crates/config/src/parsers/``) and of ``kernels/circuits/*.config.toml``: unknown
``model_type`` values are refused rather than guessed.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field, replace
from pathlib import Path
from typing import List, Optional

WEIGHT_FORMATS = ("bf16", "nvfp4", "fp8_block", "fp8_row")
KV_DTYPES = ("bf16", "fp8")
LAYER_KINDS = ("attention", "gdn", "mamba2", "mla", "kda")
FFN_KINDS = ("dense", "moe", "none")


@dataclass
class ModelConfig:
    name: str = "model"
    arch: str = "dense_gqa"            # dense_gqa | qwen_hybrid | nemotron_h | deepseek_mla
    vocab_size: int = 4096
    hidden_size: int = 256
    num_layers: int = 2
    # attention
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    rope_theta: float = 1e6
    rope_scaling: Optional[dict] = None     # HF `rope_scaling` (linear / llama3 / yarn); None = plain RoPE
    rotary_dim: int = 0                 # 0 -> head_dim; -1 -> no RoPE (Nemotron-H attention)
    rope_identity: bool = False         # keep the rotary slots of the layout but rotate by nothing (Kimi-Linear's NoPE MLA layers)
    qk_norm: bool = False
    qk_norm_full: bool = False          # the q / k RMSNorm spans all heads of the projection (MiniMax-M2), not one head
    attn_output_gate: bool = False      # q_proj emits [Q_h | G_h] per head, o = attn * sigmoid(G)
    sliding_window: int = 0
    attn_scale: float = 0.0             # softmax scale; 0 -> head_dim ** -0.5 (Gemma: query_pre_attn_scalar ** -0.5)
    window_layers: List[int] = field(default_factory=list)   # per-layer window (0 = full); empty -> sliding_window everywhere
    rope_local_theta: float = 0.0       # RoPE base of the windowed layers when it differs (Gemma 3); 0 = rope_theta
    attn_bias: bool = False             # q / k / v projections carry a bias (Qwen2 family)
    # norms
    rms_eps: float = 1e-6
    norm_plus_one: bool = False         # (1 + w) scaling (Qwen3.5 family)
    # ffn
    intermediate_size: int = 688
    ffn_act: str = "swiglu"             # swiglu | relu2 | geglu (tanh-approximated GELU gate)
    post_norms: bool = False            # Gemma / GLM-4: RMSNorm on the attention / FFN output before the residual add
    post_norm_names: str = "gemma"      # checkpoint spelling of the norms: gemma | glm | olmo2
    pre_norms: bool = True              # False: blocks read the residual stream un-normalised (OLMo 2: post-norm only)
    rope_interleaved: bool = False      # checkpoint rotates (2i, 2i+1) pairs; q / k rows are re-ordered at load
    embed_scale: float = 1.0            # embeddings are multiplied by this (Gemma: sqrt(hidden))
    final_logit_softcap: float = 0.0    # logits = cap * tanh(logits / cap); 0 = off
    residual_multiplier: float = 1.0    # Granite: a block's output is scaled by this before it joins the stream
    logits_divisor: float = 1.0         # Granite: logits are divided by this
    tie_embeddings: bool = False
    # per-layer structure
    layer_types: List[str] = field(default_factory=list)   # mixer per layer
    ffn_types: List[str] = field(default_factory=list)     # ffn per layer
    # gated delta net
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_k_dim: int = 128
    gdn_v_dim: int = 128
    conv_kernel: int = 4
    # vision input (Qwen-VL family): the tower's configuration, the placeholder token and the rotary sections
    vision: Optional[dict] = None       # HF vision_config of the checkpoint (vision.VisionConfig.from_hf)
    image_token_id: int = -1
    vision_start_token_id: int = -1
    mrope_sections: Optional[List[int]] = None      # rotary frequencies per (time, height, width) axis
    # hyper-connections: the residual stream is hc_mult fp32 copies mixed in and out of every block
    hc_mult: int = 0                    # 0 / 1 = a single residual stream
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    # sparse attention over MLA (DeepSeek sparse attention): a light indexer picks index_topk tokens per query
    index_topk: int = 0                 # 0 = dense attention
    index_n_heads: int = 64
    index_head_dim: int = 128
    # Kimi delta attention (per-channel gated delta rule)
    kda_heads: int = 0
    kda_head_dim: int = 128
    kda_gate_rank: int = 0              # inner width of the low-rank decay (f_a / f_b) and output-gate (g_a / g_b) projections; 0 = head_dim
    kda_gate_lower_bound: float = -5.0
    # mamba2
    mamba_heads: int = 0
    mamba_head_dim: int = 64
    mamba_state: int = 128
    mamba_groups: int = 8
    mamba_conv_bias: bool = True
    # moe
    num_experts: int = 0
    experts_per_token: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    shared_expert_gate: bool = False
    shared_expert_name: str = ""        # "" = by architecture ("shared_expert" for the Qwen families)
    router: str = "softmax"             # softmax | sigmoid
    router_n_group: int = 1
    router_topk_group: int = 1
    router_scaling: float = 1.0
    router_renormalize: bool = True
    first_dense_layers: int = 0
    dense_intermediate_size: int = 0    # FFN width of the leading dense layers (DeepSeek)
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_dim: int = 0
    qk_rope_dim: int = 0
    v_head_dim: int = 0
    # speculative
    mtp_layers: int = 0
    # precision
    weight_format: str = "bf16"
    kv_dtype: str = "bf16"
    kv_high_precision_layers: tuple = ()    # model layers whose KV stays bf16 when kv_dtype is fp8
    max_position: int = 32768

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = ["attention"] * self.num_layers
        if not self.ffn_types:
            self.ffn_types = ["dense"] * self.num_layers
        if self.rotary_dim == 0:
            self.rotary_dim = self.head_dim if self.arch != "deepseek_mla" else self.qk_rope_dim
        assert len(self.layer_types) == self.num_layers, "layer_types length"
        assert len(self.ffn_types) == self.num_layers, "ffn_types length"
        assert all(t in LAYER_KINDS for t in self.layer_types)
        assert all(t in FFN_KINDS for t in self.ffn_types)
        assert self.weight_format in WEIGHT_FORMATS and self.kv_dtype in KV_DTYPES

    # ---- derived sizes
    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim * (2 if self.attn_output_gate else 1)

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def gdn_qk_size(self) -> int:
        return self.gdn_k_heads * self.gdn_k_dim

    @property
    def gdn_v_size(self) -> int:
        return self.gdn_v_heads * self.gdn_v_dim

    @property
    def mamba_inner(self) -> int:
        return self.mamba_heads * self.mamba_head_dim

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_inner + 2 * self.mamba_groups * self.mamba_state

    def attention_layers(self) -> List[int]:
        return [i for i, t in enumerate(self.layer_types) if t in ("attention", "mla")]

    def kv_bytes_per_token(self) -> int:
        e = 1 if self.kv_dtype == "fp8" else 2
        n = 0
        for t in self.layer_types:
            if t == "attention":
                n += 2 * self.num_kv_heads * self.head_dim * e
            elif t == "mla":
                n += (self.kv_lora_rank + self.qk_rope_dim) * e
        return n + self.mtp_layers * 2 * self.num_kv_heads * self.head_dim * e * (self.arch != "deepseek_mla")

    def param_count(self) -> int:
        """Approximate parameter count (linear layers + embeddings)."""
        h = self.hidden_size
        n = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        for lt, ft in zip(self.layer_types, self.ffn_types):
            if lt == "attention":
                n += h * (self.q_size + 2 * self.kv_size) + self.num_heads * self.head_dim * h
            elif lt == "gdn":
                n += h * (2 * self.gdn_qk_size + 2 * self.gdn_v_size + 2 * self.gdn_v_heads) + self.gdn_v_size * h
            elif lt == "kda":
                hd, r = self.kda_heads * self.kda_head_dim, self.kda_gate_rank or self.kda_head_dim
                n += 4 * h * hd + 2 * (h * r + r * hd) + h * self.kda_heads
            elif lt == "mamba2":
                n += h * (2 * self.mamba_inner + 2 * self.mamba_groups * self.mamba_state + self.mamba_heads)
                n += self.mamba_inner * h
            elif lt == "mla":
                qh = self.qk_nope_dim + self.qk_rope_dim
                n += h * self.q_lora_rank + self.q_lora_rank * self.num_heads * qh
                n += h * (self.kv_lora_rank + self.qk_rope_dim)
                n += self.kv_lora_rank * self.num_heads * (self.qk_nope_dim + self.v_head_dim)
                n += self.num_heads * self.v_head_dim * h
            mult = 3 if self.ffn_act == "swiglu" else 2
            if ft == "dense":
                n += mult * h * (self.dense_intermediate_size or self.intermediate_size)
            elif ft == "moe":
                n += self.num_experts * mult * h * self.moe_intermediate_size + h * self.num_experts
                n += self.num_shared_experts * mult * h * self.moe_intermediate_size
        return n

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_json(s: str) -> "ModelConfig":
        return ModelConfig(**json.loads(s))

    def scaled(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


# ----------------------------------------------------------------------------- presets
def tiny_dense(**kw) -> ModelConfig:
    """Tiny dense Qwen3-style decoder that runs on CPU in fp32-equivalent precision: 2 layers,
    hidden 256, 4 q / 2 kv heads of 64, SwiGLU 688, vocab 4096, tied embeddings."""
    base = dict(name="tiny-dense", arch="dense_gqa", vocab_size=4096, hidden_size=256, num_layers=2,
                num_heads=4, num_kv_heads=2, head_dim=64, rope_theta=1e6, intermediate_size=688,
                tie_embeddings=True, rms_eps=1e-6, qk_norm=True, max_position=2048)
    base.update(kw)
    return ModelConfig(**base)


def dense_27b_nvfp4(**kw) -> ModelConfig:
    """Dense ~27B decoder: 64 layers, hidden 5120, 40 q / 8 kv heads of 128, SwiGLU 17408,
    vocab 151936, NVFP4 weights (bf16 embeddings and lm_head), fp8 KV, one MTP layer."""
    base = dict(name="dense-27b-nvfp4", arch="dense_gqa", vocab_size=151936, hidden_size=5120,
                num_layers=64, num_heads=40, num_kv_heads=8, head_dim=128, rope_theta=1e6,
                intermediate_size=17408, tie_embeddings=False, qk_norm=True, mtp_layers=1,
                weight_format="nvfp4", kv_dtype="fp8", max_position=32768)
    base.update(kw)
    return ModelConfig(**base)


def qwen_hybrid_moe_35b(**kw) -> ModelConfig:
    """Hybrid GDN + gated attention MoE, ~35B total / ~3B active, FP8 128x128 block weights:
    40 layers in a 3:1 pattern, hidden 2048, GDN 16 value heads x 128 (16 key heads), conv 4;
    attention 16 q / 2 kv heads of 256 with an output gate; 256 experts top-8 softmax + 1 shared
    expert with a sigmoid gate, expert FFN 512."""
    L = kw.pop("num_layers", 40)
    base = dict(name="qwen-hybrid-moe-35b-fp8", arch="qwen_hybrid", vocab_size=151936, hidden_size=2048,
                num_layers=L, num_heads=16, num_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7,
                qk_norm=True, attn_output_gate=True, norm_plus_one=True,
                layer_types=[("attention" if (i + 1) % 4 == 0 else "gdn") for i in range(L)],
                ffn_types=["moe"] * L, gdn_k_heads=16, gdn_v_heads=16, gdn_k_dim=128, gdn_v_dim=128,
                conv_kernel=4, num_experts=256, experts_per_token=8, moe_intermediate_size=512,
                num_shared_experts=1, shared_expert_gate=True, router="softmax", mtp_layers=0,
                weight_format="fp8_block", kv_dtype="bf16", intermediate_size=512)
    base.update(kw)
    return ModelConfig(**base)


def nemotron_h_8b(**kw) -> ModelConfig:
    """Nemotron-H style hybrid, ~8B, FP8 per-row weights: 52 layers, each one mixer *or* one MLP
    (24 Mamba2 mixers with 128 heads x 64, state 128, 8 groups, conv 4; 4 attention layers with
    32 q / 8 kv heads of 128, no RoPE; 24 squared-ReLU MLPs of 21504), hidden 4096, vocab 131072."""
    # 52 blocks = 28 mixers (24 Mamba2 + 4 attention) + 24 MLPs. A layer here is one mixer plus
    # the MLP block that follows it, if any; the Mamba2 mixer right before each attention
    # block has none ("...M*-..." in the block pattern).
    n_mix = kw.pop("num_layers", 28)
    attn_at = {4 + 6 * j for j in range(4)} if n_mix == 28 else {n_mix // 2}
    layer_types = ["attention" if i in attn_at else "mamba2" for i in range(n_mix)]
    ffn_types = ["none" if (i + 1) in attn_at else "dense" for i in range(n_mix)]
    base = dict(name="nemotron-h-8b-fp8", arch="nemotron_h", vocab_size=131072, hidden_size=4096,
                num_layers=len(layer_types), num_heads=32, num_kv_heads=8, head_dim=128, rotary_dim=-1,
                layer_types=layer_types, ffn_types=ffn_types, intermediate_size=21504, ffn_act="relu2",
                mamba_heads=128, mamba_head_dim=64, mamba_state=128, mamba_groups=8, conv_kernel=4,
                weight_format="fp8_row", kv_dtype="bf16", rms_eps=1e-5, max_position=16384)
    base.update(kw)
    return ModelConfig(**base)


def deepseek_v3_671b(**kw) -> ModelConfig:
    """DeepSeek-V3 shaped MLA MoE: 61 layers (first 3 dense, FFN 18432), hidden 7168, MLA 128
    heads (q_lora 1536, kv_lora 512, nope 128, rope 64, v 128), 256 routed experts top-8 with a
    sigmoid group-limited router (8 groups, top-4) + 1 shared expert, expert FFN 2048,
    vocab 129280, one MTP layer, FP8 128x128 block weights."""
    L = kw.pop("num_layers", 61)
    fd = kw.pop("first_dense_layers", 3)
    base = dict(name="deepseek-v3-671b-fp8", arch="deepseek_mla", vocab_size=129280, hidden_size=7168,
                num_layers=L, num_heads=128, num_kv_heads=128, head_dim=192, rope_theta=10000.0,
                layer_types=["mla"] * L, ffn_types=["dense"] * fd + ["moe"] * (L - fd),
                first_dense_layers=fd, dense_intermediate_size=18432, intermediate_size=18432,
                q_lora_rank=1536, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64, v_head_dim=128,
                num_experts=256, experts_per_token=8, moe_intermediate_size=2048, num_shared_experts=1,
                router="sigmoid", router_n_group=8, router_topk_group=4, router_scaling=2.5,
                mtp_layers=1, weight_format="fp8_block", kv_dtype="bf16", max_position=16384)
    base.update(kw)
    return ModelConfig(**base)


def tiny_hybrid_moe(**kw) -> ModelConfig:
    """Four-layer instance of the hybrid GDN + gated-attention MoE family (tests, smoke runs)."""
    base = dict(num_layers=4, hidden_size=512, num_heads=4, num_kv_heads=2, gdn_k_heads=4, gdn_v_heads=4,
                num_experts=8, experts_per_token=2, moe_intermediate_size=256, intermediate_size=256,
                vocab_size=4096, max_position=1024, name="tiny-hybrid-moe")
    base.update(kw)
    return qwen_hybrid_moe_35b(**base)


def tiny_nemotron_h(**kw) -> ModelConfig:
    """Four-mixer instance of the Mamba2 + attention hybrid family (tests, smoke runs)."""
    base = dict(num_layers=4, hidden_size=512, num_heads=8, num_kv_heads=2, intermediate_size=1024,
                mamba_heads=16, mamba_groups=2, vocab_size=4096, max_position=1024, name="tiny-nemotron-h")
    base.update(kw)
    return nemotron_h_8b(**base)


def tiny_dense_hc(**kw) -> ModelConfig:
    """The tiny dense model with a four-stream hyper-connection highway (tests, smoke runs)."""
    base = dict(hc_mult=4, hc_sinkhorn_iters=4, name="tiny-dense-hc")
    base.update(kw)
    return tiny_dense(**base)


def tiny_kimi_linear(**kw) -> ModelConfig:
    """Four-layer instance of the Kimi-Linear family: three Kimi-delta-attention layers per full-attention
    layer, MoE feed-forward (tests, smoke runs)."""
    base = dict(num_layers=4, hidden_size=512, num_heads=4, num_kv_heads=2, gdn_k_heads=0, gdn_v_heads=0,
                kda_heads=4, kda_head_dim=128, kda_gate_rank=64,
                layer_types=["kda", "kda", "kda", "attention"],
                num_experts=8, experts_per_token=2, moe_intermediate_size=256, intermediate_size=256,
                vocab_size=4096, max_position=1024, name="tiny-kimi-linear")
    base.update(kw)
    return qwen_hybrid_moe_35b(**base)


PRESETS = {
    "tiny-dense": tiny_dense,
    "tiny-kimi-linear": tiny_kimi_linear,
    "tiny-dense-hc": tiny_dense_hc,
    "tiny-hybrid-moe": tiny_hybrid_moe,
    "tiny-nemotron-h": tiny_nemotron_h,
    "dense-27b-nvfp4": dense_27b_nvfp4,
    "qwen-hybrid-moe-35b-fp8": qwen_hybrid_moe_35b,
    "nemotron-h-8b-fp8": nemotron_h_8b,
    "deepseek-v3-671b-fp8": deepseek_v3_671b,
}


def preset(name: str, **kw) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[name](**kw)


# ----------------------------------------------------------------------------- HF config.json
_HF_ARCH = {
    "llama": "dense_gqa", "qwen2": "dense_gqa", "qwen3": "dense_gqa", "mistral": "dense_gqa",
    "granite": "dense_gqa", "olmo2": "dense_gqa", "minimax_m2": "dense_gqa", "glm4": "dense_gqa", "gemma3_text": "dense_gqa", "gemma3": "dense_gqa", "gemma2": "dense_gqa",
    "phi3": "dense_gqa", "qwen3_moe": "dense_gqa", "qwen2_moe": "dense_gqa", "mixtral": "dense_gqa",
    "qwen3_5": "qwen_hybrid", "qwen3_5_moe": "qwen_hybrid", "qwen3_next": "qwen_hybrid",
    "qwen3_5_text": "qwen_hybrid", "qwen3_5_moe_text": "qwen_hybrid",
    "nemotron_h": "nemotron_h", "deepseek_v3": "deepseek_mla", "deepseek_v2": "deepseek_mla",
    "kimi_k2": "deepseek_mla",          # Kimi K2 checkpoints use the DeepSeek-V3 architecture and tensor names
    "deepseek_v32": "deepseek_mla",     # DeepSeek-V3.2: V3 + the sparse-attention indexer
    "kimi_linear": "deepseek_mla",      # Kimi-Linear: Kimi-delta-attention layers + (NoPE) MLA layers, DeepSeek-style MoE
}


# vision-language wrappers -> the text stack they carry (tensor names under model.language_model. are
# unwrapped by weights/remap.py)
_HF_VISION = {"qwen2_vl": "qwen2", "qwen2_5_vl": "qwen2", "qwen2_vl_text": "qwen2", "qwen2_5_vl_text": "qwen2",
              "qwen3_vl": "qwen3", "qwen3_vl_text": "qwen3"}


def detect_weight_format(qc: Optional[dict]) -> str:
    """quantization_config -> serving weight format
    (crates/model-layers/src/quant_format/mod.rs:61-138, weight_map/nvfp4_detect.rs:23-38)."""
    if not qc:
        return "bf16"
    method = str(qc.get("quant_method", "")).lower()
    algo = str(qc.get("quant_algo", "")).upper()
    fmt = str(qc.get("format", "")).lower()
    if method == "modelopt":
        return "nvfp4" if "NVFP4" in algo else ("fp8_row" if "FP8" in algo else "bf16")
    if method == "compressed-tensors":
        if "float-quantized" in fmt or "fp8" in fmt:
            return "fp8_row"
        return "nvfp4"
    if method == "fp8":
        return "fp8_block" if qc.get("weight_block_size") else "fp8_row"
    raise ValueError(f"unsupported quant_method {method!r}")


def from_hf_config(cfg: dict, name: str = "model") -> ModelConfig:
    """Map a HF ``config.json`` dict (text stack) to ModelConfig; refuses unknown model types."""
    outer = cfg
    if "text_config" in cfg:
        inner = dict(cfg["text_config"])
        inner.setdefault("quantization_config", cfg.get("quantization_config"))
        cfg = inner
    mt = cfg.get("model_type", "")
    vision_kw = {}
    if outer.get("vision_config") and (outer.get("model_type", "") in _HF_VISION or mt in _HF_VISION):
        rs = cfg.get("rope_scaling") or outer.get("rope_scaling") or {}
        vision_kw = dict(vision=dict(outer["vision_config"]), image_token_id=int(outer.get("image_token_id", -1)),
                         vision_start_token_id=int(outer.get("vision_start_token_id", -1)),
                         mrope_sections=list(rs["mrope_section"]) if rs.get("mrope_section") else None)
        if mt in _HF_VISION:
            mt = _HF_VISION[mt]
        if (rs.get("type") or rs.get("rope_type")) in ("mrope", "default"):
            cfg = dict(cfg)
            cfg["rope_scaling"] = None                     # the sections only say which axis a frequency follows
    if mt not in _HF_ARCH:
        raise ValueError(f"unsupported model_type {mt!r}")
    arch = _HF_ARCH[mt]
    h = cfg["hidden_size"]
    L = cfg["num_hidden_layers"]
    heads = cfg.get("num_attention_heads", 1)
    kw = dict(name=name, arch=arch, vocab_size=cfg["vocab_size"], hidden_size=h, num_layers=L,
              num_heads=heads, num_kv_heads=cfg.get("num_key_value_heads", heads),
              head_dim=cfg.get("head_dim", h // heads), rope_theta=float(cfg.get("rope_theta", 1e4)), rope_scaling=cfg.get("rope_scaling"),
              rms_eps=float(cfg.get("rms_norm_eps", cfg.get("layer_norm_epsilon", 1e-6))),
              intermediate_size=cfg.get("intermediate_size", 0),
              tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
              max_position=int(cfg.get("max_position_embeddings", 32768)),
              weight_format=detect_weight_format(cfg.get("quantization_config")),
              mtp_layers=int(cfg.get("mtp_num_hidden_layers", cfg.get("num_nextn_predict_layers", 0)) or 0))
    if arch == "dense_gqa":
        kw["qk_norm"] = mt in ("qwen3", "qwen3_moe")
        kw["attn_bias"] = bool(cfg.get("attention_bias", cfg.get("qkv_bias", mt in ("qwen2", "qwen2_moe"))))
        kw["sliding_window"] = int(cfg.get("sliding_window") or 0) if cfg.get("use_sliding_window") else 0
        if mt in ("gemma3_text", "gemma3", "gemma2"):
            if cfg.get("attn_logit_softcapping"):
                raise ValueError("attention logit soft-capping (Gemma 2) is not supported")
            act = cfg.get("hidden_activation", cfg.get("hidden_act", "gelu_pytorch_tanh"))
            if act not in ("gelu_pytorch_tanh", "gelu_tanh"):
                raise ValueError(f"unsupported Gemma activation {act!r}")
            win = int(cfg.get("sliding_window") or 0)
            lt = cfg.get("layer_types")
            if lt is None:
                pat = int(cfg.get("sliding_window_pattern", 6) or 6)
                lt = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(L)]
            kw.update(norm_plus_one=True, post_norms=True, ffn_act="geglu", qk_norm=mt != "gemma2",
                      embed_scale=float(h) ** 0.5, tie_embeddings=bool(cfg.get("tie_word_embeddings", True)),
                      attn_scale=float(cfg.get("query_pre_attn_scalar", kw["head_dim"])) ** -0.5,
                      window_layers=[win if t == "sliding_attention" else 0 for t in lt], sliding_window=0,
                      rope_local_theta=float(cfg.get("rope_local_base_freq", 0.0) or 0.0),
                      final_logit_softcap=float(cfg.get("final_logit_softcapping") or 0.0))
        if mt == "granite":
            kw.update(embed_scale=float(cfg.get("embedding_multiplier", 1.0)), attn_scale=float(cfg.get("attention_multiplier", 0.0) or 0.0),
                      residual_multiplier=float(cfg.get("residual_multiplier", 1.0)),
                      logits_divisor=float(cfg.get("logits_scaling", 1.0) or 1.0),
                      attn_bias=bool(cfg.get("attention_bias", False)))
        if mt == "olmo2":
            kw.update(post_norms=True, post_norm_names="olmo2", pre_norms=False, qk_norm=True, qk_norm_full=True,
                      attn_bias=bool(cfg.get("attention_bias", False)))
        if mt == "minimax_m2":
            if cfg.get("shared_intermediate_size"):
                raise ValueError("MiniMax shared experts are not supported")
            kw.update(qk_norm=bool(cfg.get("use_qk_norm", True)), qk_norm_full=cfg.get("qk_norm_type", "per_layer") == "per_layer",
                      rotary_dim=int(cfg.get("rotary_dim", kw["head_dim"])), ffn_types=["moe"] * L,
                      num_experts=int(cfg.get("num_local_experts", 0)), experts_per_token=int(cfg.get("num_experts_per_tok", 8)),
                      moe_intermediate_size=cfg.get("intermediate_size", 0),
                      router="sigmoid" if cfg.get("scoring_func", "sigmoid") == "sigmoid" else "softmax",
                      router_renormalize=True, router_scaling=float(cfg.get("routed_scaling_factor", 1.0)))
        if mt == "glm4":
            kw.update(post_norms=True, post_norm_names="glm", rope_interleaved=True,
                      attn_bias=bool(cfg.get("attention_bias", True)),
                      rotary_dim=int(kw["head_dim"] * float(cfg.get("partial_rotary_factor", 0.5))))
        if mt == "phi3":
            rs = cfg.get("rope_scaling")
            if rs and str(rs.get("type", rs.get("rope_type", ""))).lower() in ("longrope", "su"):
                raise ValueError("phi3 longrope scaling is not supported")
            prf = float(cfg.get("partial_rotary_factor", 1.0))
            if prf < 1.0:
                kw["rotary_dim"] = int(kw["head_dim"] * prf)
        if mt in ("qwen3_moe", "qwen2_moe"):
            step = int(cfg.get("decoder_sparse_step", 1) or 1)
            only = set(cfg.get("mlp_only_layers") or [])
            ne = int(cfg.get("num_experts", 0))
            kw.update(ffn_types=["moe" if ne and i not in only and (i + 1) % step == 0 else "dense" for i in range(L)],
                      num_experts=ne, experts_per_token=cfg.get("num_experts_per_tok", 8),
                      moe_intermediate_size=cfg.get("moe_intermediate_size", 768), router="softmax",
                      router_renormalize=bool(cfg.get("norm_topk_prob", mt == "qwen3_moe")))
            if mt == "qwen2_moe" and cfg.get("shared_expert_intermediate_size", 0):
                mi = kw["moe_intermediate_size"]
                sh = int(cfg["shared_expert_intermediate_size"])
                if sh % mi:
                    raise ValueError("shared expert width must be a multiple of the routed expert width")
                kw.update(num_shared_experts=sh // mi, shared_expert_gate=True, shared_expert_name="shared_expert")
        if mt == "mixtral":
            kw.update(ffn_types=["moe"] * L, num_experts=int(cfg.get("num_local_experts", 8)),
                      experts_per_token=int(cfg.get("num_experts_per_tok", 2)),
                      moe_intermediate_size=cfg.get("intermediate_size", 0), router="softmax", router_renormalize=True)
    elif arch == "qwen_hybrid":
        lt = cfg.get("layer_types")
        interval = cfg.get("full_attention_interval", 4)
        if lt is None:
            lt = ["full_attention" if (i + 1) % interval == 0 else "linear_attention" for i in range(L)]
        if cfg.get("linear_conv_kernel_dim", 4) != 4:
            raise ValueError("linear_conv_kernel_dim must be 4")
        kw.update(layer_types=["attention" if t == "full_attention" else "gdn" for t in lt],
                  qk_norm=True, attn_output_gate=bool(cfg.get("attn_output_gate", True)), norm_plus_one=True,
                  rotary_dim=int(cfg.get("head_dim", h // heads) * cfg.get("partial_rotary_factor", 0.25)),
                  gdn_k_heads=cfg.get("linear_num_key_heads", 16), gdn_v_heads=cfg.get("linear_num_value_heads", 32),
                  gdn_k_dim=cfg.get("linear_key_head_dim", 128), gdn_v_dim=cfg.get("linear_value_head_dim", 128))
        ne = cfg.get("num_experts", 0)
        if ne:
            kw.update(ffn_types=["moe"] * L, num_experts=ne, experts_per_token=cfg.get("num_experts_per_tok", 8),
                      moe_intermediate_size=cfg.get("moe_intermediate_size", 512),
                      num_shared_experts=1 if cfg.get("shared_expert_intermediate_size", 0) else 0,
                      shared_expert_gate=True, router="softmax",
                      router_renormalize=bool(cfg.get("norm_topk_prob", True)))
    elif arch == "nemotron_h":
        pat = cfg.get("hybrid_override_pattern", "")
        lt, ft = [], []
        for ch in pat:
            if ch == "M":
                lt.append("mamba2"); ft.append("none")
            elif ch == "*":
                lt.append("attention"); ft.append("none")
            elif ch in "-E":
                # an MLP/MoE block: attach to the previous mixer when it has no FFN yet
                if lt and ft[-1] == "none":
                    ft[-1] = "dense" if ch == "-" else "moe"
                else:
                    lt.append("mamba2"); ft.append("dense" if ch == "-" else "moe")
        kw.update(layer_types=lt, ffn_types=ft, num_layers=len(lt), rotary_dim=-1, ffn_act="relu2",
                  mamba_heads=cfg.get("mamba_num_heads", 128), mamba_head_dim=cfg.get("mamba_head_dim", 64),
                  mamba_state=cfg.get("ssm_state_size", 128), mamba_groups=cfg.get("n_groups", 8),
                  conv_kernel=cfg.get("conv_kernel", 4))
    else:
        fd = cfg.get("first_k_dense_replace", 0)
        kw.update(layer_types=["mla"] * L, ffn_types=["dense"] * fd + ["moe"] * (L - fd), first_dense_layers=fd,
                  dense_intermediate_size=cfg.get("intermediate_size", 0),
                  q_lora_rank=cfg.get("q_lora_rank") or 0, kv_lora_rank=cfg.get("kv_lora_rank", 512),
                  qk_nope_dim=cfg.get("qk_nope_head_dim", 128), qk_rope_dim=cfg.get("qk_rope_head_dim", 64),
                  v_head_dim=cfg.get("v_head_dim", 128), head_dim=cfg.get("qk_nope_head_dim", 128) + cfg.get("qk_rope_head_dim", 64),
                  num_experts=cfg.get("n_routed_experts", 0), experts_per_token=cfg.get("num_experts_per_tok", 8),
                  moe_intermediate_size=cfg.get("moe_intermediate_size", 2048),
                  num_shared_experts=cfg.get("n_shared_experts", 0),
                  router="sigmoid" if cfg.get("scoring_func", "softmax") == "sigmoid" else "softmax",
                  router_n_group=cfg.get("n_group", 1), router_topk_group=cfg.get("topk_group", 1),
                  router_scaling=float(cfg.get("routed_scaling_factor", 1.0)),
                  router_renormalize=bool(cfg.get("norm_topk_prob", True)))
        if cfg.get("index_topk"):
            kw.update(index_topk=int(cfg["index_topk"]), index_n_heads=int(cfg.get("index_n_heads", 64)),
                      index_head_dim=int(cfg.get("index_head_dim", 128)))
        if mt == "kimi_linear":
            la = cfg.get("linear_attn_config") or {}
            kda_layers = {int(i) - 1 for i in la.get("kda_layers", [])}            # the checkpoint counts layers from 1
            if not kda_layers:
                raise ValueError("kimi_linear needs linear_attn_config.kda_layers")
            conv = int(la.get("short_conv_kernel_size", 4))
            kw.update(layer_types=["kda" if i in kda_layers else "mla" for i in range(L)],
                      kda_heads=int(la.get("num_heads", heads)), kda_head_dim=int(la.get("head_dim", 128)),
                      kda_gate_rank=int(la.get("gate_rank", 0) or 0), conv_kernel=conv,
                      kda_gate_lower_bound=float(la.get("gate_lower_bound", -5.0)),
                      rope_identity=bool(cfg.get("mla_use_nope", False)),
                      num_experts=cfg.get("num_experts", cfg.get("n_routed_experts", 0)),
                      experts_per_token=cfg.get("num_experts_per_token", cfg.get("num_experts_per_tok", 8)),
                      num_shared_experts=cfg.get("num_shared_experts", cfg.get("n_shared_experts", 0)),
                      router="sigmoid" if cfg.get("moe_router_activation_func", cfg.get("scoring_func", "sigmoid")) == "sigmoid" else "softmax",
                      router_n_group=cfg.get("num_expert_group", cfg.get("n_group", 1)),
                      router_topk_group=cfg.get("topk_group", 1),
                      router_renormalize=bool(cfg.get("moe_renormalize", cfg.get("norm_topk_prob", True))))
    kw.update(vision_kw)
    return ModelConfig(**kw)


def load_hf_config(path) -> ModelConfig:
    p = Path(path)
    return from_hf_config(json.loads((p / "config.json").read_text()), name=p.name)
