"""Open a checkpoint directory: HF ``config.json`` (or the engine's own ``engine_config.json``
written by ``write_checkpoint``) + safetensors shards -> (ModelConfig, TensorSource)."""
from __future__ import annotations

import json
from pathlib import Path

from ..config.model_config import ModelConfig, from_hf_config
from .fast_source import open_source


def open_checkpoint(path, device="cpu"):
    p = Path(path)
    ggufs = [p] if p.is_file() and p.suffix == ".gguf" else (sorted(p.glob("*.gguf")) if p.is_dir() else [])
    if ggufs and not list(p.glob("*.safetensors") if p.is_dir() else []):
        from .gguf import GgufSource
        src = GgufSource(ggufs[0])
        return src.cfg, src
    src = open_source(p, device=device)
    eng = p / "engine_config.json"
    if eng.exists():
        cfg = ModelConfig.from_json(eng.read_text())
    else:
        hf = json.loads((p / "config.json").read_text())
        cfg = from_hf_config(hf, name=p.name)
        from .remap import family_source
        src = family_source(src, hf)          # Mixtral / fused-projection / wrapped-text-stack naming
    return cfg, src
