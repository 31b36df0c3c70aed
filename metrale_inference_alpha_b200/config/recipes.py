"""Serving recipes: a YAML file that names a model and the serve options that go with it, so a
deployment is one file instead of a command line. Keys are the `serve` option names (dashes or
underscores); unknown keys are refused. Role of the reference's recipe YAML parsing
(``crates/config/src/recipes``).

    model: /models/dense-27b-nvfp4
    served_model_name: dense-27b
    max_num_seqs: 128
    max_model_len: 32768
    speculative: mtp
    tool_call_parser: hermes
    lora_adapters: {sql: /adapters/sql, support: /adapters/support}
    env: {METRALE_PDL: "2"}
"""
from __future__ import annotations

from typing import Dict, List

import yaml


def load_recipe(path: str) -> Dict[str, object]:
    with open(path) as f:
        d = yaml.safe_load(f) or {}
    if not isinstance(d, dict) or "model" not in d:
        raise ValueError(f"{path}: a recipe is a mapping with at least a `model` key")
    return {str(k).replace("-", "_"): v for k, v in d.items()}


def recipe_to_argv(recipe: Dict[str, object], known_options: List[str]) -> List[str]:
    """Translate a recipe into `serve` arguments; `known_options` are the parser's option strings."""
    from ..utils.levers import LEVERS
    known = {o.lstrip("-").replace("-", "_"): o for o in known_options}
    argv: List[str] = []
    for key, val in recipe.items():
        if key == "env":
            bad = [k for k in val if k.startswith("METRALE_") and k not in LEVERS]
            if bad:
                raise ValueError(f"recipe sets undeclared levers: {bad}")
            continue
        if key == "lora_adapters":
            for name, p in (val or {}).items():
                argv += ["--lora-adapter", f"{name}={p}"]
            continue
        if key not in known:
            raise ValueError(f"recipe key {key!r} is not a serve option")
        opt = known[key]
        if isinstance(val, bool):
            argv.append(opt if val else opt.replace("--", "--no-", 1))
        elif isinstance(val, (list, tuple)):
            for v in val:
                argv += [opt, str(v)]
        elif val is not None:
            argv += [opt, str(val)]
    return argv
