"""Checkpoint name dialects. The loader asks for tensors by one canonical naming (the Llama / Qwen
layout: ``model.layers.N.self_attn.{q,k,v,o}_proj``, ``mlp.{gate,up,down}_proj``,
``mlp.gate`` + ``mlp.experts.E.*``); ``MappedSource`` answers those names from checkpoints that
spell them differently:

* multimodal wrappers whose text stack sits under ``model.language_model.`` /
  ``language_model.model.`` (prefix found by probing for the embedding table);
* Mixtral: ``block_sparse_moe.gate`` and experts ``w1`` / ``w3`` / ``w2``;
* Phi-3 style fused projections: ``qkv_proj`` rows split into q | k | v, ``gate_up_proj`` rows
  into gate | up (every tensor of the linear that has one row per output feature is sliced, so
  per-row quantisation scales follow their rows).

Role of the per-family weight maps of the reference (``crates/model-arch/src/*/weight_map*``).
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from .source import TensorSource

# canonical name -> (checkpoint name, optional (row_lo, row_hi, total_rows))
Resolve = Callable[[str], Optional[Tuple[str, Optional[Tuple[int, int, int]]]]]


class MappedSource(TensorSource):
    def __init__(self, inner: TensorSource, resolvers: List[Resolve], prefix: Tuple[str, str] = ("", "")):
        self.inner, self.resolvers, self.prefix = inner, resolvers, prefix
        self.quant_config = inner.quant_config

    def _locate(self, name: str):
        cands = [(name, None)]
        for r in self.resolvers:
            hit = r(name)
            if hit is not None:
                cands.insert(0, hit)
        old, new = self.prefix
        out = []
        for n, sl in cands:
            if old and n.startswith(old):
                out.append((new + n[len(old):], sl))
            out.append((n, sl))
        for n, sl in out:
            if self.inner.has(n):
                return n, sl
        return None

    def has(self, name: str) -> bool:
        return self._locate(name) is not None

    def get(self, name: str) -> torch.Tensor:
        hit = self._locate(name)
        if hit is None:
            raise KeyError(name)
        n, sl = hit
        t = self.inner.get(n)
        if sl is not None:
            lo, hi, total = sl
            if t.dim() >= 1 and t.shape[0] == total:
                t = t[lo:hi]
            elif t.dim() >= 1 and t.shape[0] not in (1,) and total % t.shape[0] == 0 and t.shape[0] != total:
                # row-blocked scales (one row of scales per `blk` output rows)
                blk = total // t.shape[0]
                if lo % blk or hi % blk:
                    raise ValueError(f"{n}: fused-projection split {lo}:{hi} cuts a scale block of {blk} rows")
                t = t[lo // blk:hi // blk]
        return t

    def names(self) -> Iterable[str]:
        return self.inner.names()

    def __getattr__(self, k):                   # cfg, metadata, ... of the wrapped source
        return getattr(self.inner, k)


def _mixtral(name: str):
    if name.endswith(".mlp.gate.e_score_correction_bias"):        # MiniMax keeps the routing bias beside the gate
        return name[:-len("mlp.gate.e_score_correction_bias")] + "block_sparse_moe.e_score_correction_bias", None
    m = re.match(r"(.*\.)mlp\.(gate\.weight|experts\.(\d+)\.(gate|up|down)_proj\.(.+))$", name)
    if not m:
        return None
    if m.group(2) == "gate.weight":
        return m.group(1) + "block_sparse_moe.gate.weight", None
    w = {"gate": "w1", "up": "w3", "down": "w2"}[m.group(4)]
    return f"{m.group(1)}block_sparse_moe.experts.{m.group(3)}.{w}.{m.group(5)}", None


def _fused(q_rows: int, kv_rows: int, inter: int) -> Resolve:
    qkv_total = q_rows + 2 * kv_rows
    spans = {"q": (0, q_rows), "k": (q_rows, q_rows + kv_rows), "v": (q_rows + kv_rows, qkv_total)}

    def resolve(name: str):
        m = re.match(r"(.*\.self_attn\.)([qkv])_proj\.(.+)$", name)
        if m:
            lo, hi = spans[m.group(2)]
            return f"{m.group(1)}qkv_proj.{m.group(3)}", (lo, hi, qkv_total)
        m = re.match(r"(.*\.mlp\.)(gate|up)_proj\.(.+)$", name)
        if m:
            lo = 0 if m.group(2) == "gate" else inter
            return f"{m.group(1)}gate_up_proj.{m.group(3)}", (lo, lo + inter, 2 * inter)
        return None
    return resolve


def _find_prefix(src: TensorSource) -> Tuple[str, str]:
    if src.has("model.embed_tokens.weight"):
        return "", ""
    for new in ("model.language_model.", "language_model.model.", "model.text_model.", "text_model."):
        if src.has(new + "embed_tokens.weight"):
            return "model.", new
    return "", ""


def family_source(src: TensorSource, hf_cfg: Optional[dict]) -> TensorSource:
    """Wraps `src` when its naming differs from the canonical one; returns it unchanged otherwise."""
    cfg = dict(hf_cfg or {})
    if "text_config" in cfg:
        cfg = dict(cfg["text_config"])
    mt = cfg.get("model_type", "")
    resolvers: List[Resolve] = []
    if mt in ("mixtral", "minimax_m2"):
        resolvers.append(_mixtral)
    if mt in ("phi3", "phi4", "glm4") or src.has("model.layers.0.self_attn.qkv_proj.weight") \
            or src.has("model.layers.0.mlp.gate_up_proj.weight"):
        h = cfg.get("hidden_size", 0)
        heads = cfg.get("num_attention_heads", 1)
        hd = cfg.get("head_dim", h // max(1, heads))
        kvh = cfg.get("num_key_value_heads", heads)
        resolvers.append(_fused(heads * hd, kvh * hd, cfg.get("intermediate_size", 0)))
    prefix = _find_prefix(src)
    # lm_head of wrapped text stacks may live at the top level or under the wrapper
    if not resolvers and prefix == ("", ""):
        return src
    ms = MappedSource(src, resolvers, prefix)
    if prefix[1] and not src.has("lm_head.weight"):
        for cand in ("language_model.lm_head.weight", "model.lm_head.weight"):
            if src.has(cand):
                base = cand[:-len("weight")]
                ms.resolvers.append(lambda n, b=base: (b + n[len("lm_head."):], None) if n.startswith("lm_head.") else None)
                break
    return ms
