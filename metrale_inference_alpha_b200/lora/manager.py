"""Multi-adapter LoRA serving: adapters live in fixed device slots, every token row of a step
carries its sequence's slot (-1 = base model), and the delta of each targeted projection is added
to the base projection's bf16 output by two small kernels (``ops/csrc/lora.cu``: shrink + expand).

Checkpoint layout accepted: PEFT (``adapter_config.json`` with ``r`` / ``lora_alpha`` /
``target_modules``; ``adapter_model.safetensors`` with
``base_model.model.model.layers.{i}.{self_attn|mlp}.{q,k,v,o,down}_proj.lora_{A,B}.weight``).
Targets served: q/k/v (addressed inside the fused qkv output), o, down. gate/up adapters are
refused at load time: the fused SwiGLU epilogue has no place to add them.

The prefix cache keys its roots by adapter name, so KV computed under one adapter is never reused
under another. Role of the reference's ``crates/model-layers/src/lora`` + ``lora_bgmv.cu`` and the
LoRA swap path of ``crates/model-engine``.
"""
from __future__ import annotations

import ctypes as C
import json
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import _native

MAX_RANK = 64
TARGETS = ("q", "k", "v", "o", "down")
_native.register_optional("mb_lora_shrink", [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                             C.c_int, C.c_int, C.c_void_p, C.c_void_p])
_native.register_optional("mb_lora_expand", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                             C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p])
_NAME = re.compile(r"layers\.(\d+)\.(?:self_attn|mlp)\.(q|k|v|o|down|gate|up)_proj\.lora_(A|B)\.weight$")


@dataclass
class LoraAdapter:
    name: str
    rank: int
    alpha: float
    # (layer, target) -> (A [rank, K], B [N, rank])
    weights: Dict[Tuple[int, str], Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)

    @property
    def scale(self) -> float:
        return self.alpha / self.rank

    @classmethod
    def from_tensors(cls, name: str, tensors: Dict[str, torch.Tensor], rank: int, alpha: float) -> "LoraAdapter":
        ad = cls(name, rank, alpha)
        halves: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
        for key, t in tensors.items():
            m = _NAME.search(key)
            if not m:
                continue
            layer, target, which = int(m.group(1)), m.group(2), m.group(3)
            if target not in TARGETS:
                raise ValueError(f"adapter {name!r}: LoRA on {target}_proj is not served (fused SwiGLU epilogue)")
            halves.setdefault((layer, target), {})[which] = t
        for k, h in halves.items():
            if "A" not in h or "B" not in h:
                raise ValueError(f"adapter {name!r}: {k} lacks lora_A or lora_B")
            if h["A"].shape[0] != rank or h["B"].shape[1] != rank or rank > MAX_RANK:
                raise ValueError(f"adapter {name!r}: {k} has rank {h['A'].shape[0]} / {h['B'].shape[1]}, declared {rank}")
            ad.weights[k] = (h["A"].to(torch.bfloat16), h["B"].to(torch.bfloat16))
        return ad

    @classmethod
    def from_dir(cls, name: str, path) -> "LoraAdapter":
        from safetensors.torch import load_file
        p = Path(path)
        cfg = json.loads((p / "adapter_config.json").read_text())
        return cls.from_tensors(name, load_file(str(p / "adapter_model.safetensors")), int(cfg["r"]),
                                float(cfg.get("lora_alpha", cfg["r"])))


class LoraManager:
    """Fixed pool of adapter slots with stacked per-(layer, target) tensors on the device."""

    def __init__(self, num_layers: int, dims: Dict[str, Tuple[int, int]], max_adapters: int = 8,
                 max_rank: int = 16, device="cpu", max_rows: int = 8192):
        """dims[target] = (K, N) of that projection on this rank."""
        assert max_rank <= MAX_RANK
        self.device, self.L, self.dims = torch.device(device), num_layers, dims
        self.max_adapters, self.rank = max_adapters, max_rank
        self.A = {(l, t): torch.zeros(max_adapters, max_rank, dims[t][0], dtype=torch.bfloat16, device=device)
                  for l in range(num_layers) for t in dims}
        self.B = {(l, t): torch.zeros(max_adapters, dims[t][1], max_rank, dtype=torch.bfloat16, device=device)
                  for l in range(num_layers) for t in dims}
        self.scales = torch.zeros(max_adapters, dtype=torch.float32, device=device)
        self.slots: Dict[str, int] = {}
        self.present: Dict[int, set] = {}
        self._tmp = torch.zeros(max_rows, MAX_RANK, dtype=torch.float32, device=device)

    def bytes(self) -> int:
        return sum(t.numel() * 2 for t in self.A.values()) + sum(t.numel() * 2 for t in self.B.values())

    def names(self) -> List[str]:
        return sorted(self.slots)

    def slot_of(self, name: Optional[str]) -> int:
        return -1 if not name else self.slots[name]

    def load(self, ad: LoraAdapter) -> int:
        if ad.name in self.slots:
            slot = self.slots[ad.name]
        else:
            free = [s for s in range(self.max_adapters) if s not in self.slots.values()]
            if not free:
                raise RuntimeError(f"all {self.max_adapters} adapter slots are in use; unload one first")
            slot = free[0]
        if ad.rank > self.rank:
            raise ValueError(f"adapter rank {ad.rank} exceeds the pool's max_rank {self.rank}")
        for (l, t), (a, b) in ad.weights.items():
            K, N = self.dims[t]
            if a.shape[1] != K or b.shape[0] != N:
                raise ValueError(f"adapter {ad.name!r} layer {l} {t}: shapes {tuple(a.shape)} / {tuple(b.shape)} "
                                 f"do not match the model ({K} -> {N})")
        for key in self.A:
            self.A[key][slot].zero_()
            self.B[key][slot].zero_()
        for (l, t), (a, b) in ad.weights.items():
            self.A[(l, t)][slot, :ad.rank].copy_(a)
            self.B[(l, t)][slot, :, :ad.rank].copy_(b)
        self.scales[slot] = ad.scale
        self.slots[ad.name] = slot
        self.present[slot] = set(ad.weights)
        return slot

    def unload(self, name: str) -> None:
        slot = self.slots.pop(name)
        self.present.pop(slot, None)
        self.scales[slot] = 0.0

    def active(self, layer: int, target: str) -> bool:
        return any((layer, target) in p for p in self.present.values())

    # ------------------------------------------------------------------ application
    def apply(self, out: torch.Tensor, x: torch.Tensor, layer: int, target: str, rows: torch.Tensor,
              col0: int = 0) -> None:
        """out[:, col0:col0+N] += scale * B (A x) for the rows whose slot is >= 0 (in place)."""
        if not self.active(layer, target):
            return
        A, B = self.A[(layer, target)], self.B[(layer, target)]
        M, N = x.shape[0], B.shape[1]
        if not x.is_cuda:
            sel = rows[:M].long()
            on = sel >= 0
            if not bool(on.any()):
                return
            idx = sel.clamp(min=0)
            t = torch.einsum("mk,mrk->mr", x.float(), A[idx].float())
            d = torch.einsum("mr,mnr->mn", t, B[idx].float()) * self.scales[idx][:, None]
            d = torch.where(on[:, None], d, torch.zeros_like(d))
            out[:, col0:col0 + N] = (out[:, col0:col0 + N].float() + d).to(out.dtype)
            return
        from ..ops import _count, _ptr, _stream, runtime
        L = _native.lib()
        assert out.dtype == torch.bfloat16 and x.dtype == torch.bfloat16 and M <= self._tmp.shape[0]
        st = _ptr(runtime(x.device).status)
        _native.check(L.mb_lora_shrink(_ptr(x), x.stride(0), _ptr(A), _ptr(rows), _ptr(self._tmp), M, x.shape[1],
                                       self.rank, self.max_adapters, st, _stream()), "lora_shrink")
        _native.check(L.mb_lora_expand(_ptr(self._tmp), _ptr(B), _ptr(rows), _ptr(self.scales), _ptr(out),
                                       out.stride(0), col0, M, N, self.rank, self.max_adapters, _stream()), "lora_expand")
        _count(2)
