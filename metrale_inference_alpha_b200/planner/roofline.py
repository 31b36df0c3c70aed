"""Hardware planner: the decode step of a model as a list of ops with their algorithmic bytes and
FLOPs, and a roofline estimate per op and per step against measured device peaks. Pure (no GPU, no
IO besides the optional peaks file), so it serves `doctor`, capacity planning and the comparison
of measured kernel times with what the bytes allow. Role of the reference's circuit op graphs and
hardware planner with rooflines (``crates/circuit/src/hardware``, ``kernels/DEVICES.toml``), in
reduced form: the graph is derived from the model config instead of a declarative circuit file.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

from ..config.model_config import ModelConfig

WEIGHT_BYTES = {"nvfp4": 0.5 + 1.0 / 16.0, "fp8_block": 1.0, "fp8_row": 1.0, "bf16": 2.0}
ACT_BYTES = {"nvfp4": 0.5 + 1.0 / 16.0, "fp8_block": 1.0, "fp8_row": 1.0, "bf16": 2.0}
# dense tensor-core peak relative to bf16 for each operand kind
FLOP_SCALE = {"nvfp4": 4.0, "fp8_block": 2.0, "fp8_row": 2.0, "bf16": 1.0}


@dataclass
class DevicePeaks:
    hbm_gbs: float = 6650.0            # measured copy bandwidth (fallback figures of this pool)
    bf16_tflops: float = 1590.0
    launch_us: float = 2.5             # floor of a dependent kernel launch inside a CUDA graph
    source: str = "fallback"


def load_peaks(path: Optional[str] = None) -> DevicePeaks:
    for p in filter(None, [path, os.environ.get("METRALE_PEAKS_JSON"), "MEASURED_PEAKS.json"]):
        if os.path.exists(p):
            d = json.load(open(p))
            return DevicePeaks(float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                               source=f"measured ({p})")
    return DevicePeaks()


@dataclass
class LayerOp:
    name: str
    count: int                  # launches per step
    bytes: float                # algorithmic bytes per launch
    flops: float                # per launch
    kind: str = "bf16"          # operand kind (scales the tensor-core peak)

    def time_us(self, peaks: DevicePeaks) -> float:
        mem = self.bytes / (peaks.hbm_gbs * 1e3)
        cmp_ = self.flops / (peaks.bf16_tflops * FLOP_SCALE.get(self.kind, 1.0) * 1e6)
        return max(mem, cmp_, peaks.launch_us)


def _gemm(name, count, M, N, K, fmt, out_bytes=2.0) -> LayerOp:
    return LayerOp(name, count, N * K * WEIGHT_BYTES[fmt] + M * K * ACT_BYTES[fmt] + M * N * out_bytes,
                   2.0 * M * N * K, fmt)


def decode_step_ops(cfg: ModelConfig, batch: int, ctx: int, tp: int = 1) -> List[LayerOp]:
    """One decode step (one new token per sequence) of `cfg` on one rank of a `tp`-way shard."""
    h, D, fmt = cfg.hidden_size, cfg.head_dim, cfg.weight_format
    hq, hkv = max(1, cfg.num_heads // tp), max(1, cfg.num_kv_heads // tp)
    kv_b = 1.0 if cfg.kv_dtype == "fp8" else 2.0
    layer_types = cfg.layer_types or ["attention"] * cfg.num_layers
    ffn_types = cfg.ffn_types or ["dense"] * cfg.num_layers
    n_attn = sum(t == "attention" for t in layer_types)
    n_mla = sum(t == "mla" for t in layer_types)
    n_rec = sum(t in ("gdn", "mamba2") for t in layer_types)
    n_dense = sum(t == "dense" for t in ffn_types)
    n_moe = sum(t == "moe" for t in ffn_types)
    M = batch
    ops: List[LayerOp] = [LayerOp("embed", 1, M * h * 2.0 * 2, 0.0)]
    L = cfg.num_layers
    ops.append(LayerOp("rmsnorm+quant", 2 * L, M * h * (2.0 + ACT_BYTES[fmt]), 4.0 * M * h))
    if n_attn:
        ops.append(_gemm("qkv", n_attn, M, (hq + 2 * hkv) * D, h, fmt))
        ops.append(LayerOp("qk-norm+rope+kv-write", n_attn, M * (hq + 2 * hkv) * D * 2.0 * 2, 0.0))
        ops.append(LayerOp("paged attention", n_attn, M * ctx * hkv * D * 2 * kv_b + 2 * M * hq * D * 2.0,
                           4.0 * M * hq * D * ctx, "bf16"))
        ops.append(_gemm("o_proj", n_attn, M, h, hq * D, fmt))
    if n_mla:
        row = (cfg.kv_lora_rank + cfg.qk_rope_dim) * 2.0
        ops.append(LayerOp("mla attention", n_mla, M * ctx * row, 4.0 * M * hq * ctx * (cfg.kv_lora_rank + cfg.qk_rope_dim)))
    if n_rec:
        state = (cfg.gdn_v_heads or cfg.mamba_heads or 1) * (cfg.gdn_k_dim or cfg.mamba_head_dim or 1) * \
                (cfg.gdn_v_dim or cfg.mamba_state or 1) * 4.0 / tp
        ops.append(LayerOp("recurrent state update", n_rec, 2.0 * M * state, 6.0 * M * state / 4.0))
    if n_dense:
        inter = cfg.intermediate_size // tp
        ops.append(_gemm("gate_up+swiglu", n_dense, M, 2 * inter, h, fmt, out_bytes=ACT_BYTES[fmt] / 2))
        ops.append(_gemm("down", n_dense, M, h, inter, fmt))
    if n_moe:
        e_act = min(cfg.num_experts, M * cfg.experts_per_token)          # experts touched by the batch
        inter = cfg.moe_intermediate_size
        w = e_act * 3 * inter * h * WEIGHT_BYTES[fmt] / tp
        ops.append(LayerOp("moe experts", n_moe, w + M * cfg.experts_per_token * (h + inter) * 2.0,
                           2.0 * M * cfg.experts_per_token * 3 * inter * h / tp, fmt))
        ops.append(LayerOp("moe route+sort+combine", 3 * n_moe, M * cfg.num_experts * 4.0, 0.0))
    ops.append(_gemm("lm_head", 1, M, cfg.vocab_size // tp, h, "bf16", out_bytes=4.0))
    ops.append(LayerOp("argmax / sample", 1, M * cfg.vocab_size / tp * 4.0, 0.0))
    return ops


def estimate(cfg: ModelConfig, batch: int, ctx: int, tp: int = 1, peaks: Optional[DevicePeaks] = None) -> Dict[str, object]:
    peaks = peaks or load_peaks()
    ops = decode_step_ops(cfg, batch, ctx, tp)
    rows, total_us, bytes_total, flops_total, launches = [], 0.0, 0.0, 0.0, 0
    for op in ops:
        t = op.time_us(peaks)
        rows.append({"op": op.name, "count": op.count, "us_each": round(t, 2), "us_total": round(t * op.count, 1),
                     "mbytes_each": round(op.bytes / 1e6, 3), "bound": "launch" if t == peaks.launch_us else
                     ("memory" if op.bytes / (peaks.hbm_gbs * 1e3) >= t - 1e-9 else "compute")})
        total_us += t * op.count
        bytes_total += op.bytes * op.count
        flops_total += op.flops * op.count
        launches += op.count
    pure_mem_ms = bytes_total / (peaks.hbm_gbs * 1e6)
    return {"model": cfg.name, "batch": batch, "ctx": ctx, "tp": tp, "peaks": peaks.source, "ops": rows,
            "launches": launches, "step_ms_roofline_per_op": round(total_us / 1e3, 3),
            "step_ms_bytes_only": round(pure_mem_ms, 3), "tok_s_upper_bound": round(batch / (pure_mem_ms / 1e3), 1),
            "gbytes_per_step": round(bytes_total / 1e9, 3), "tflop_per_step": round(flops_total / 1e12, 3)}
