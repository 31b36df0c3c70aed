"""Model hot-swap: the HTTP listener, its routes and the scheduler thread stay; the engine behind
them is replaced once the running requests have drained.

Every route closure and the scheduler thread hold an `EngineProxy`, which forwards attribute access
to the engine currently loaded; `AsyncEngine.request_swap` performs the replacement on the scheduler
thread between ticks, so no step ever runs on two models and requests that arrive during the swap
are answered by the new model. The old engine's device memory is released before the new model's
KV cache is sized. Role of the reference's ``crates/server/src/main_modules/model_swap.rs``.
"""
from __future__ import annotations

import dataclasses
from typing import Optional


class Proxy:
    def __init__(self, engine):
        object.__setattr__(self, "_target", engine)
        object.__setattr__(self, "swaps", 0)

    def target(self):
        return object.__getattribute__(self, "_target")

    def swap(self, engine) -> None:
        object.__setattr__(self, "_target", engine)
        object.__setattr__(self, "swaps", object.__getattribute__(self, "swaps") + 1)

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "_target"), name)

    def __setattr__(self, name, value):
        setattr(object.__getattribute__(self, "_target"), name, value)


EngineProxy = Proxy


def build_like(old_engine, model, tokenizer_dir: Optional[str] = None, **overrides):
    """A new engine with the old one's arguments and another model (a preset name or a checkpoint
    directory), plus its tokenizer when the directory has one."""
    from ..engine.llm_engine import LLMEngine
    from .tokenizer import load_tokenizer
    args = dataclasses.replace(old_engine.args, model=model, **overrides)
    tp = getattr(old_engine, "tp", None)
    # the old engine must be unreachable before the new one sizes its KV cache: the caller drops it
    eng = LLMEngine(args, tp=tp if getattr(tp, "size", 1) > 1 else None)
    tok = load_tokenizer(tokenizer_dir if tokenizer_dir else (model if isinstance(model, str) else None), eng.cfg.vocab_size)
    return eng, tok
