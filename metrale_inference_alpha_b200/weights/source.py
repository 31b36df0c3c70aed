"""Where checkpoint tensors come from.

``SafetensorsSource`` reads a HF checkpoint directory (sharded ``*.safetensors`` with the usual
``model.safetensors.index.json``); ``SyntheticSource`` produces random-init tensors *in the
same HF layouts and names* (NVFP4 ModelOpt / compressed-tensors, FP8 128x128 block, FP8
per-row, bf16), generated lazily per tensor so a 27B or 671B-shaped model never exists in
fp32 at once. ``write_checkpoint`` materialises a source to disk (tests, small models).
Role of the reference's ``crates/model-weights`` (mmap safetensors loader, preflight) and of
``crates/core/src/safetensors.rs``.
"""
from __future__ import annotations

import hashlib
import json
import re
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..ops import reference as ref


class TensorSource:
    def has(self, name: str) -> bool:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def names(self) -> Iterable[str]:
        raise NotImplementedError

    quant_config: Optional[dict] = None


class DictSource(TensorSource):
    def __init__(self, tensors: Dict[str, torch.Tensor], quant_config: Optional[dict] = None):
        self.t = tensors
        self.quant_config = quant_config

    def has(self, name):
        return name in self.t

    def get(self, name):
        return self.t[name]

    def names(self):
        return self.t.keys()


class SafetensorsSource(TensorSource):
    def __init__(self, path, device="cpu"):
        from safetensors import safe_open
        self.path = Path(path)
        self.device = str(device)
        self._open = safe_open
        self._index: Dict[str, Path] = {}
        idx = self.path / "model.safetensors.index.json"
        if idx.exists():
            for name, shard in json.loads(idx.read_text())["weight_map"].items():
                self._index[name] = self.path / shard
        else:
            for f in sorted(self.path.glob("*.safetensors")):
                with safe_open(str(f), framework="pt") as h:
                    for name in h.keys():
                        self._index[name] = f
        self._handles = {}
        cfgp = self.path / "config.json"
        if cfgp.exists():
            c = json.loads(cfgp.read_text())
            self.quant_config = c.get("quantization_config") or c.get("text_config", {}).get("quantization_config")
        hq = self.path / "hf_quant_config.json"
        if self.quant_config is None and hq.exists():
            q = json.loads(hq.read_text()).get("quantization", {})
            self.quant_config = {"quant_method": "modelopt", "quant_algo": q.get("quant_algo", "")}

    def _h(self, f: Path):
        if f not in self._handles:
            self._handles[f] = self._open(str(f), framework="pt", device=self.device)
        return self._handles[f]

    def has(self, name):
        return name in self._index

    def get(self, name):
        t = self._h(self._index[name]).get_tensor(name)
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        return t

    def names(self):
        return self._index.keys()

    def preflight(self, required: Iterable[str]) -> List[str]:
        """Names that are required but absent (checkpoint preflight)."""
        return [n for n in required if n not in self._index]


def _seed_for(name: str, seed: int) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


class SyntheticSource(TensorSource):
    """Random N(0, std) weights in HF checkpoint layout for `cfg`. Each tensor is a pure
    function of (seed, name), so every rank of a tensor-parallel job sees the same checkpoint."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu",
                 nvfp4_dialect: str = "modelopt"):
        self.cfg, self.seed, self.std, self.device = cfg, seed, std, torch.device(device)
        self.dialect = nvfp4_dialect
        self.shapes: Dict[str, tuple] = {}
        self.kinds: Dict[str, str] = {}
        self._describe()
        fmt = cfg.weight_format
        if fmt == "nvfp4":
            self.quant_config = ({"quant_method": "modelopt", "quant_algo": "NVFP4"} if nvfp4_dialect == "modelopt"
                                 else {"quant_method": "compressed-tensors", "format": "nvfp4-pack-quantized"})
        elif fmt == "fp8_block":
            self.quant_config = {"quant_method": "fp8", "weight_block_size": [128, 128]}
        elif fmt == "fp8_row":
            self.quant_config = {"quant_method": "fp8"}
        self._cache_name = None
        self._cache_val: Dict[str, torch.Tensor] = {}

    # ---- layout description
    def _lin(self, prefix: str, n: int, k: int, quant: bool = True):
        self.shapes[prefix] = (n, k)
        self.kinds[prefix] = self.cfg.weight_format if quant else "bf16"

    def _vec(self, name: str, n, kind="norm"):
        self.shapes[name] = (n,) if isinstance(n, int) else tuple(n)
        self.kinds[name] = kind

    def _attn(self, p: str):
        c = self.cfg
        self._lin(f"{p}.q_proj", c.q_size, c.hidden_size)
        self._lin(f"{p}.k_proj", c.kv_size, c.hidden_size)
        self._lin(f"{p}.v_proj", c.kv_size, c.hidden_size)
        self._lin(f"{p}.o_proj", c.hidden_size, c.num_heads * c.head_dim)
        if c.qk_norm:
            self._vec(f"{p}.q_norm.weight", c.q_size if c.qk_norm_full else c.head_dim)
            self._vec(f"{p}.k_norm.weight", c.kv_size if c.qk_norm_full else c.head_dim)
        if c.attn_bias:
            self._vec(f"{p}.q_proj.bias", c.q_size, "bias")
            self._vec(f"{p}.k_proj.bias", c.kv_size, "bias")
            self._vec(f"{p}.v_proj.bias", c.kv_size, "bias")

    def _ffn(self, p: str, inter: int, names=("gate_proj", "up_proj", "down_proj")):
        c = self.cfg
        if c.ffn_act in ("swiglu", "geglu"):
            self._lin(f"{p}.{names[0]}", inter, c.hidden_size)
        self._lin(f"{p}.{names[1]}", inter, c.hidden_size)
        self._lin(f"{p}.{names[2]}", c.hidden_size, inter)

    def _describe(self):
        c = self.cfg
        if c.arch == "nemotron_h":
            return self._describe_nemotron()
        self._lin("model.embed_tokens", c.vocab_size, c.hidden_size, quant=False)
        if not c.tie_embeddings:
            self._lin("lm_head", c.vocab_size, c.hidden_size, quant=False)
        self._vec("model.norm.weight", c.hidden_size)
        for i in range(c.num_layers):
            self._layer(f"model.layers.{i}", c.layer_types[i], c.ffn_types[i], i)
        for j in range(c.mtp_layers):
            self._lin("mtp.fc", c.hidden_size, 2 * c.hidden_size, quant=False)
            self._vec("mtp.pre_fc_norm_embedding.weight", c.hidden_size)
            self._vec("mtp.pre_fc_norm_hidden.weight", c.hidden_size)
            self._vec("mtp.norm.weight", c.hidden_size)
            lt = "mla" if c.arch == "deepseek_mla" else "attention"
            ft = "moe" if c.num_experts else "dense"
            self._layer(f"mtp.layers.{j}", lt, ft, c.num_layers + j)

    def _layer(self, p: str, lt: str, ft: str, idx: int):
        c = self.cfg
        if c.pre_norms:
            self._vec(f"{p}.input_layernorm.weight", c.hidden_size)
        if lt == "attention":
            self._attn(f"{p}.self_attn")
        elif lt == "gdn":
            q = f"{p}.linear_attn"
            self._lin(f"{q}.in_proj_qkv", 2 * c.gdn_qk_size + c.gdn_v_size, c.hidden_size)
            self._lin(f"{q}.in_proj_z", c.gdn_v_size, c.hidden_size)
            self._lin(f"{q}.in_proj_b", c.gdn_v_heads, c.hidden_size, quant=False)
            self._lin(f"{q}.in_proj_a", c.gdn_v_heads, c.hidden_size, quant=False)
            self._vec(f"{q}.conv1d.weight", (2 * c.gdn_qk_size + c.gdn_v_size, 1, c.conv_kernel), "conv")
            self._vec(f"{q}.A_log", c.gdn_v_heads, "alog")
            self._vec(f"{q}.dt_bias", c.gdn_v_heads, "bias")
            self._vec(f"{q}.norm.weight", c.gdn_v_dim, "ones")
            self._lin(f"{q}.out_proj", c.hidden_size, c.gdn_v_size)
        elif lt == "kda":
            q = f"{p}.self_attn"
            hd, r = c.kda_heads * c.kda_head_dim, c.kda_gate_rank or c.kda_head_dim
            for n in "qkv":
                self._lin(f"{q}.{n}_proj", hd, c.hidden_size)
                self._vec(f"{q}.{n}_conv1d.weight", (hd, 1, c.conv_kernel), "conv")
            self._lin(f"{q}.f_a_proj", r, c.hidden_size, quant=False)
            self._lin(f"{q}.f_b_proj", hd, r, quant=False)
            self._lin(f"{q}.g_a_proj", r, c.hidden_size, quant=False)
            self._lin(f"{q}.g_b_proj", hd, r, quant=False)
            self._lin(f"{q}.b_proj", c.kda_heads, c.hidden_size, quant=False)
            self._vec(f"{q}.A_log", c.kda_heads, "alog")
            self._vec(f"{q}.dt_bias", hd, "bias")
            self._vec(f"{q}.o_norm.weight", c.kda_head_dim, "ones")
            self._lin(f"{q}.o_proj", c.hidden_size, hd)
        elif lt == "mla":
            q = f"{p}.self_attn"
            qh = c.qk_nope_dim + c.qk_rope_dim
            if c.q_lora_rank:
                self._lin(f"{q}.q_a_proj", c.q_lora_rank, c.hidden_size)
                self._vec(f"{q}.q_a_layernorm.weight", c.q_lora_rank)
                self._lin(f"{q}.q_b_proj", c.num_heads * qh, c.q_lora_rank)
            else:
                self._lin(f"{q}.q_proj", c.num_heads * qh, c.hidden_size)
            self._lin(f"{q}.kv_a_proj_with_mqa", c.kv_lora_rank + c.qk_rope_dim, c.hidden_size)
            self._vec(f"{q}.kv_a_layernorm.weight", c.kv_lora_rank)
            self._lin(f"{q}.kv_b_proj", c.num_heads * (c.qk_nope_dim + c.v_head_dim), c.kv_lora_rank)
            self._lin(f"{q}.o_proj", c.hidden_size, c.num_heads * c.v_head_dim)
            if c.index_topk > 0:
                self._lin(f"{q}.indexer.wq_b", c.index_n_heads * c.index_head_dim, c.q_lora_rank or c.hidden_size, quant=False)
                self._lin(f"{q}.indexer.wk", c.index_head_dim, c.hidden_size, quant=False)
                self._lin(f"{q}.indexer.weights_proj", c.index_n_heads, c.hidden_size, quant=False)
                self._vec(f"{q}.indexer.k_norm.weight", c.index_head_dim, "ones")
                self._vec(f"{q}.indexer.k_norm.bias", c.index_head_dim, "bias")
        if c.hc_mult > 1:
            mix = (2 + c.hc_mult) * c.hc_mult
            for site in ("attn_hc", "ffn_hc"):
                self._vec(f"{p}.{site}.fn", (mix, c.hc_mult * c.hidden_size), "small")
                self._vec(f"{p}.{site}.scale", 3, "ones")
                self._vec(f"{p}.{site}.base", mix, "bias")
        if ft != "none":
            self._vec(f"{p}.post_attention_layernorm.weight", c.hidden_size)
            if c.post_norms and c.post_norm_names == "olmo2":
                self._vec(f"{p}.post_feedforward_layernorm.weight", c.hidden_size)
            elif c.post_norms and c.post_norm_names == "glm":
                self._vec(f"{p}.post_self_attn_layernorm.weight", c.hidden_size)
                self._vec(f"{p}.post_mlp_layernorm.weight", c.hidden_size)
            elif c.post_norms:
                self._vec(f"{p}.pre_feedforward_layernorm.weight", c.hidden_size)
                self._vec(f"{p}.post_feedforward_layernorm.weight", c.hidden_size)
        if ft == "dense":
            inter = c.dense_intermediate_size if (c.dense_intermediate_size and idx < c.first_dense_layers) else c.intermediate_size
            self._ffn(f"{p}.mlp", inter)
        elif ft == "moe":
            self._lin(f"{p}.mlp.gate", c.num_experts, c.hidden_size, quant=False)
            if c.router == "sigmoid":
                self._vec(f"{p}.mlp.gate.e_score_correction_bias", c.num_experts, "bias")
            for e in range(c.num_experts):
                self._ffn(f"{p}.mlp.experts.{e}", c.moe_intermediate_size)
            if c.num_shared_experts:
                sp = c.shared_expert_name or ("shared_expert" if c.arch == "qwen_hybrid" else "shared_experts")
                self._ffn(f"{p}.mlp.{sp}", c.moe_intermediate_size * c.num_shared_experts)
                if c.shared_expert_gate:
                    self._lin(f"{p}.mlp.shared_expert_gate", 1, c.hidden_size, quant=False)

    def nemotron_blocks(self):
        """HF block index of each layer's mixer and MLP (blocks are numbered separately there)."""
        c = self.cfg
        out, b = [], 0
        for i in range(c.num_layers):
            mixer = b
            b += 1
            mlp = None
            if c.ffn_types[i] != "none":
                mlp = b
                b += 1
            out.append((mixer, mlp))
        return out

    def _describe_nemotron(self):
        c = self.cfg
        self._lin("backbone.embeddings", c.vocab_size, c.hidden_size, quant=False)
        self._lin("lm_head", c.vocab_size, c.hidden_size, quant=False)
        self._vec("backbone.norm_f.weight", c.hidden_size)
        for i, (mb, fb) in enumerate(self.nemotron_blocks()):
            p = f"backbone.layers.{mb}"
            self._vec(f"{p}.norm.weight", c.hidden_size)
            if c.layer_types[i] == "mamba2":
                self._lin(f"{p}.mixer.in_proj", 2 * c.mamba_inner + 2 * c.mamba_groups * c.mamba_state + c.mamba_heads,
                          c.hidden_size)
                self._vec(f"{p}.mixer.conv1d.weight", (c.mamba_conv_dim, 1, c.conv_kernel), "conv")
                self._vec(f"{p}.mixer.conv1d.bias", c.mamba_conv_dim, "bias")
                self._vec(f"{p}.mixer.A_log", c.mamba_heads, "alog")
                self._vec(f"{p}.mixer.D", c.mamba_heads, "ones")
                self._vec(f"{p}.mixer.dt_bias", c.mamba_heads, "bias")
                self._vec(f"{p}.mixer.norm.weight", c.mamba_inner, "ones")
                self._lin(f"{p}.mixer.out_proj", c.hidden_size, c.mamba_inner)
            else:
                self._attn(f"{p}.mixer")
            if fb is not None:
                q = f"backbone.layers.{fb}"
                self._vec(f"{q}.norm.weight", c.hidden_size)
                self._ffn(f"{q}.mixer", c.intermediate_size)

    # ---- tensor generation
    def _rand(self, name: str, shape, std: float) -> torch.Tensor:
        g = torch.Generator(device=self.device).manual_seed(_seed_for(name, self.seed))
        return torch.randn(*shape, generator=g, device=self.device, dtype=torch.float32) * std

    def _linear_tensors(self, prefix: str) -> Dict[str, torch.Tensor]:
        if self._cache_name == prefix:
            return self._cache_val
        n, k = self.shapes[prefix]
        w = self._rand(prefix + ".weight", (n, k), self.std)
        kind = self.kinds[prefix]
        out: Dict[str, torch.Tensor] = {}
        if kind == "bf16":
            out["weight"] = w.to(torch.bfloat16)
        elif kind == "nvfp4":
            q, sf, g = ref.quantize_nvfp4(w, per_row_global=False)
            if self.dialect == "modelopt":
                out["weight"], out["weight_scale"] = q, sf
                out["weight_scale_2"] = g.reshape(()).float()
            else:
                out["weight_packed"], out["weight_scale"] = q, sf
                out["weight_global_scale"] = (1.0 / g).reshape(1).float()
        elif kind == "fp8_block":
            q, s = ref.quantize_fp8_block128(w)
            out["weight"], out["weight_scale_inv"] = q, s
        elif kind == "fp8_row":
            q, s = ref.quantize_fp8_rowwise(w)
            out["weight"], out["weight_scale"] = q, s
        self._cache_name, self._cache_val = prefix, out
        return out

    def _split(self, name: str):
        m = re.match(r"^(.*)\.(weight|weight_packed|weight_scale|weight_scale_2|weight_scale_inv|weight_global_scale)$", name)
        if m and m.group(1) in self.shapes and len(self.shapes[m.group(1)]) == 2 and m.group(1) in self.kinds \
                and self.kinds[m.group(1)] in ("bf16", "nvfp4", "fp8_block", "fp8_row"):
            return m.group(1), m.group(2)
        return None, None

    def has(self, name: str) -> bool:
        if name in self.shapes and self.kinds[name] not in ("bf16", "nvfp4", "fp8_block", "fp8_row"):
            return True
        prefix, suffix = self._split(name)
        if prefix is None:
            return False
        kind = self.kinds[prefix]
        valid = {"bf16": {"weight"},
                 "nvfp4": {"weight", "weight_scale", "weight_scale_2"} if self.dialect == "modelopt"
                 else {"weight_packed", "weight_scale", "weight_global_scale"},
                 "fp8_block": {"weight", "weight_scale_inv"}, "fp8_row": {"weight", "weight_scale"}}[kind]
        return suffix in valid

    def get(self, name: str) -> torch.Tensor:
        if name in self.shapes and self.kinds[name] not in ("bf16", "nvfp4", "fp8_block", "fp8_row"):
            kind, shape = self.kinds[name], self.shapes[name]
            if kind == "norm":
                # (1 + w) models store w around 0, plain-weight models around 1
                base = 0.0 if self.cfg.norm_plus_one else 1.0
                return (base + self._rand(name, shape, 0.02)).to(torch.bfloat16)
            if kind == "ones":
                return (1.0 + self._rand(name, shape, 0.02)).to(torch.bfloat16)
            if kind == "conv":
                return self._rand(name, shape, 0.3).to(torch.bfloat16)
            if kind == "alog":
                return (self._rand(name, shape, 0.3)).float()
            if kind == "bias":
                return self._rand(name, shape, 0.1).float()
            if kind == "small":
                return self._rand(name, shape, 0.02).to(torch.bfloat16)
        prefix, suffix = self._split(name)
        if prefix is None or not self.has(name):
            raise KeyError(name)
        return self._linear_tensors(prefix)[suffix]

    def names(self):
        out = []
        for p, kind in self.kinds.items():
            if kind in ("bf16", "nvfp4", "fp8_block", "fp8_row"):
                for suf in ("weight", "weight_packed", "weight_scale", "weight_scale_2", "weight_scale_inv",
                            "weight_global_scale"):
                    if self.has(f"{p}.{suf}"):
                        out.append(f"{p}.{suf}")
            else:
                out.append(p)
        return out


def write_checkpoint(src: TensorSource, cfg: ModelConfig, path, shard_bytes: int = 1 << 30) -> Path:
    """Write `src` as a sharded safetensors checkpoint with an index and an engine config."""
    from safetensors.torch import save_file
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    shard: Dict[str, torch.Tensor] = {}
    size, shard_id, weight_map, files = 0, 0, {}, []

    def flush():
        nonlocal shard, size, shard_id
        if not shard:
            return
        fname = f"model-{shard_id:05d}.safetensors"
        save_file(shard, str(path / fname))
        files.append(fname)
        for n in shard:
            weight_map[n] = fname
        shard, size, shard_id = {}, 0, shard_id + 1

    for name in src.names():
        t = src.get(name).detach().cpu().contiguous()
        shard[name] = t
        size += t.numel() * t.element_size()
        if size >= shard_bytes:
            flush()
    flush()
    (path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    (path / "engine_config.json").write_text(cfg.to_json())
    (path / "config.json").write_text(json.dumps({"quantization_config": src.quant_config, "engine": True}))
    return path
