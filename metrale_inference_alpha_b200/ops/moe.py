"""Mixture-of-experts ops: router top-k and the routed-expert FFN.

CPU path (oracle): route with the reference formulas, then loop over experts.
CUDA path: ``csrc/moe.cu`` — one block per token for routing (softmax top-k, or sigmoid +
selection bias + group-limited top-k), a counting sort of (token, expert) pairs into
expert-contiguous rows with a tile work-list, then the tcgen05 grouped GEMMs over
``[experts * N, K]`` stacked weights, and a weighted un-permute that also blends the shared
expert. Reference behaviour: ``kernels/gb10/common/moe_topk.cu``, ``moe_topk_sigmoid.cu``,
``moe_permute.cu``, ``moe_w8a8_grouped_gemm.cu``, ``moe_unpermute_blend.cu``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _native, reference as ref


@dataclass
class GroupedExperts:
    """Experts stacked along N for the grouped GEMM: gate_up [E * 2I, K], down [E * H, I]."""
    gate_up: object
    down: object
    num: int
    n_gate_up: int
    n_down: int
    interleaved: bool
    shared_slot: Optional[int] = None     # local expert index of a folded-in shared expert (every token routes to it)


def stack_experts(experts) -> Optional[GroupedExperts]:
    if not experts:
        return None
    from . import concat_weights
    nvfp4 = experts[0].gate_up.fmt == "nvfp4"
    if nvfp4 and (experts[0].gate_up.N % 128 or experts[0].down.N % 128):
        # the scale factors of an NVFP4 operand are tiled by 128 rows: an expert whose row count is not a
        # multiple of that shares a tile with its neighbour, and such experts run one GEMM per active expert
        # (models/moe.py::routed_experts) instead of the grouped path
        return None
    gu = concat_weights([e.gate_up for e in experts])
    dn = concat_weights([e.down for e in experts])
    if nvfp4 and gu.data.is_cuda:
        gu.prepare_cuda()                                  # tiled scale factors, built once at load
        dn.prepare_cuda()
    return GroupedExperts(gu, dn, len(experts), experts[0].gate_up.N, experts[0].down.N,
                          experts[0].interleaved)


def route(logits: torch.Tensor, cfg, bias=None):
    """Router logits [T, E] fp32 -> (weights [T, k] fp32, expert ids [T, k] int32)."""
    k = cfg.experts_per_token
    if logits.is_cuda and _native.available() and hasattr(_native.lib(), "mb_moe_route"):
        from .moe_cuda import route_cuda
        return route_cuda(logits, cfg, bias)
    if cfg.router == "softmax":
        w, idx = ref.route_softmax_topk(logits, k, cfg.router_renormalize)
    else:
        w, idx = ref.route_sigmoid_grouped(logits, bias, k, cfg.router_n_group, cfg.router_topk_group,
                                           cfg.router_renormalize, cfg.router_scaling)
    return w.float(), idx.to(torch.int32)
