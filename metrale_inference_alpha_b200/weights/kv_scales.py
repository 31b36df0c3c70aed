"""Per-layer FP8 KV-cache scales of a checkpoint: one resolver for the three spellings exporters
use, relative to an attention prefix ``p`` (``model.layers.N.self_attn``):

    k_proj_output   p.k_proj.k_scale / p.v_proj.v_scale    ModelOpt, older llm-compressor
    attn_module     p.attn.k_scale   / p.attn.v_scale      vLLM's own Attention module name
    bare            p.k_scale        / p.v_scale           llm-compressor kv_cache_scheme

Every spelling carries the dequant multiplier amax / 448: the cache write divides by it, the
attention kernels multiply by it. A layer that uses two spellings, or has K without V, is an
error, never a silent 1.0. Role of ``crates/model-weights/src/weights/kv_scale_keys.rs:1-60``.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

SPELLINGS = (("k_proj_output", "k_proj.k_scale", "v_proj.v_scale"),
             ("attn_module", "attn.k_scale", "attn.v_scale"),
             ("bare", "k_scale", "v_scale"))


def resolve_kv_scale_keys(has, attn_prefix: str) -> Optional[Tuple[str, str, str]]:
    """(spelling, K key, V key) of the attention layer at `attn_prefix`, or None when the
    checkpoint carries no scale for it. `has(name)` tells whether a tensor exists."""
    found = []
    for name, ks, vs in SPELLINGS:
        k, v = f"{attn_prefix}.{ks}", f"{attn_prefix}.{vs}"
        hk, hv = has(k), has(v)
        if hk != hv:
            raise ValueError(f"{attn_prefix}: KV scale spelled {name!r} has {'K' if hk else 'V'} but not {'V' if hk else 'K'}")
        if hk:
            found.append((name, k, v))
    if len(found) > 1:
        raise ValueError(f"{attn_prefix}: KV scales spelled {len(found)} ways ({', '.join(f[0] for f in found)})")
    return found[0] if found else None


def load_kv_scales(source, attn_prefixes: Dict[int, str]) -> Dict[int, Tuple[float, float]]:
    """layer index -> (k_scale, v_scale) for every layer whose checkpoint carries the pair."""
    out = {}
    for li, prefix in attn_prefixes.items():
        keys = resolve_kv_scale_keys(source.has, prefix)
        if keys is None:
            continue
        _, k, v = keys
        ks, vs = float(source.get(k).float().reshape(-1)[0]), float(source.get(v).float().reshape(-1)[0])
        if not (ks > 0 and vs > 0):
            raise ValueError(f"{prefix}: non-positive KV scale ({ks}, {vs})")
        out[li] = (ks, vs)
    return out


def kv_scale_census(source, attn_prefixes: Dict[int, str]) -> Dict[str, int]:
    """How many layers use which spelling (what serve logs at start-up)."""
    census: Dict[str, int] = {}
    for prefix in attn_prefixes.values():
        keys = resolve_kv_scale_keys(source.has, prefix)
        name = keys[0] if keys else "none"
        census[name] = census.get(name, 0) + 1
    return census
