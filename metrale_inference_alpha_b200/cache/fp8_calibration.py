"""Online calibration of the per-layer FP8 KV-cache scales, for checkpoints that carry none.

The running max of |K| and |V| of every attention layer accumulates over the first
``window_tokens`` tokens the engine writes (across requests). Entries written inside the window
use a provisional scale wide enough not to clip; the step that reaches the window freezes
``scale = amax * headroom / 448`` per layer and rewrites the window's entries at that scale (an
entry is only read correctly at the scale that wrote it, and attention dequantises a
sequence's whole history with one scale). CUDA graphs stay off until the freeze, because the
scale tensors and the cache contents change under them.

Differences from the reference (``crates/model-layers/src/layers/fp8_calibration.rs:1-50``): the
max is taken inside the KV-write kernel (an atomic max per warp, no extra pass), and the
rewrite re-encodes the stored e4m3 values (value * provisional / frozen) instead of keeping a
bf16 copy of the window; the provisional scale keeps every value in e4m3's normal range, so
this costs at most one extra rounding step for the window's tokens only.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops

PROVISIONAL_SCALE = 2.0          # 2.0 * 448 covers |x| <= 896


class Fp8KvCalibration:
    def __init__(self, kv, window_tokens: int, headroom: float = 1.0):
        self.kv = kv
        self.window = int(window_tokens)
        self.headroom = max(1.0, float(headroom))
        self.layers = [i for i in range(kv.cfg.num_layers) if kv.k[i].dtype == torch.uint8]
        self.amax = {i: torch.zeros(2, dtype=torch.float32, device=kv.device) for i in self.layers}
        self.slots: List[torch.Tensor] = []
        self.observed = 0
        self.frozen = not self.layers or self.window <= 0
        if not self.frozen:
            for i in self.layers:
                kv.k_scale[i].fill_(PROVISIONAL_SCALE)
                kv.v_scale[i].fill_(PROVISIONAL_SCALE)

    def amax_for(self, layer: int):
        """The [2] accumulator the KV-write kernel of `layer` updates, or None once frozen."""
        return None if self.frozen else self.amax.get(layer)

    def after_step(self, slot_mapping: torch.Tensor) -> bool:
        """Call once per forward with that step's slot mapping. Returns True on the step that froze."""
        if self.frozen:
            return False
        live = slot_mapping[slot_mapping >= 0]
        self.slots.append(live.clone())
        self.observed += int(live.numel())
        if self.observed < self.window:
            return False
        self.freeze()
        return True

    def freeze(self) -> None:
        slots = torch.cat(self.slots) if self.slots else torch.zeros(0, dtype=torch.int64, device=self.kv.device)
        for i in self.layers:
            for which, cache, scale in ((0, self.kv.k[i], self.kv.k_scale[i]), (1, self.kv.v[i], self.kv.v_scale[i])):
                if cache is None:
                    continue
                a = float(self.amax[i][which])
                new = a * self.headroom / 448.0 if a > 0 else 1.0
                scale.fill_(new)
                if slots.numel():
                    ops.kv_rescale(cache, slots, PROVISIONAL_SCALE, scale)
        self.slots = []
        self.frozen = True
