"""Checkpoint preflight: before any tensor is read, compare what the model configuration needs
with what the checkpoint holds, and report everything that is wrong at once (missing tensors,
wrong shapes, a quantisation dialect the loader does not read) instead of failing on the first
``KeyError`` ten minutes into a load. The expected layout is the one ``SyntheticSource`` describes
for the same configuration, so the two cannot drift apart; names are asked through the family
dialect mapping (``weights/remap.py``), so Mixtral / Phi-3 / wrapped checkpoints pass as they load.

Role of the reference's ``crates/model-weights/src/preflight.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from ..config.model_config import ModelConfig
from .source import SyntheticSource, TensorSource

_WEIGHT_KEYS = ("weight", "weight_packed", "qweight")


@dataclass
class PreflightReport:
    checked: int = 0
    missing: List[str] = field(default_factory=list)
    bad_shape: List[Tuple[str, tuple, tuple]] = field(default_factory=list)     # name, found, expected
    notes: List[str] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return not self.missing and not self.bad_shape

    def summary(self, limit: int = 12) -> str:
        if self.ok:
            return f"checkpoint preflight: {self.checked} tensors present with the expected shapes"
        lines = [f"checkpoint preflight failed: {len(self.missing)} missing, {len(self.bad_shape)} with a wrong shape "
                 f"(of {self.checked} expected)"]
        lines += [f"  missing   {n}" for n in self.missing[:limit]]
        if len(self.missing) > limit:
            lines.append(f"  ... and {len(self.missing) - limit} more missing")
        lines += [f"  shape     {n}: found {tuple(f)}, expected {tuple(e)}" for n, f, e in self.bad_shape[:limit]]
        return "\n".join(lines + self.notes)


def _shape_of(src: TensorSource, name: str) -> Optional[tuple]:
    fn = getattr(src, "shape_of", None)
    if fn is not None:
        try:
            return tuple(fn(name))
        except Exception:
            pass
    try:
        return tuple(src.get(name).shape)
    except Exception:
        return None


def preflight(cfg: ModelConfig, src: TensorSource, check_shapes: bool = True, max_shape_checks: int = 4096) -> PreflightReport:
    want = SyntheticSource(cfg, seed=0)
    rep = PreflightReport()
    shape_checks = 0
    for name, shape in want.shapes.items():
        kind = want.kinds[name]
        rep.checked += 1
        if kind in ("bf16", "nvfp4", "fp8_block", "fp8_row"):          # a linear layer: `name` is its prefix
            found = next((f"{name}.{k}" for k in _WEIGHT_KEYS if src.has(f"{name}.{k}")), None)
            if found is None:
                rep.missing.append(f"{name}.weight")
                continue
            if check_shapes and shape_checks < max_shape_checks:
                shape_checks += 1
                got = _shape_of(src, found)
                n, k = shape
                ok_shapes = {(n, k), (n, k // 2)}                        # bf16 / fp8 bytes, or two fp4 values per byte
                if got is not None and tuple(got) not in ok_shapes:
                    rep.bad_shape.append((found, got, (n, k)))
        else:
            if not src.has(name):
                rep.missing.append(name)
                continue
            if check_shapes and shape_checks < max_shape_checks:
                shape_checks += 1
                got = _shape_of(src, name)
                if got is not None and tuple(got) != tuple(shape) and int(__import__("math").prod(got)) != int(__import__("math").prod(shape)):
                    rep.bad_shape.append((name, got, tuple(shape)))
    if cfg.weight_format == "nvfp4" and not any(src.has(f"{p}.weight_scale") for p in list(want.shapes)[:64]
                                               if want.kinds[p] == "nvfp4"):
        if any(want.kinds[p] == "nvfp4" for p in want.shapes):
            rep.notes.append("  note      no `.weight_scale` tensors found: the checkpoint will be quantised to NVFP4 at load")
    return rep
