"""Serving an NLLB / M2M-100 translation checkpoint on the OpenAI-shaped routes.

``serve --model <m2m_100 checkpoint> --nllb-src-lang eng_Latn --nllb-tgt-lang fra_Latn``: the prompt of
``/v1/completions`` (or the last user message of ``/v1/chat/completions``) is translated sentence by
sentence with beam search; the language pair can be overridden per request with ``src_lang`` /
``tgt_lang``. Language codes are tokens of the checkpoint's tokenizer (``eng_Latn``, ``fra_Latn``, ...).
Reference: the ``--nllb-src-lang`` / ``--nllb-tgt-lang`` serve options and the NLLB path of
``crates/model-engine``.
"""
from __future__ import annotations

import json
import re
import time
import uuid
from pathlib import Path
from typing import Any, Dict, List, Optional


def is_translation_checkpoint(path) -> bool:
    p = Path(path) / "config.json"
    try:
        return json.loads(p.read_text()).get("model_type") in ("m2m_100", "nllb")
    except (OSError, ValueError):
        return False


def open_translation_model(path, device="cpu"):
    """(NllbModel, HF config dict) from a checkpoint directory with safetensors weights."""
    from ..models.nllb import NllbConfig, NllbModel
    from ..weights.fast_source import open_source
    hf = json.loads((Path(path) / "config.json").read_text())
    src = open_source(Path(path), device="cpu")
    return NllbModel(NllbConfig.from_hf(hf), {n: src.get(n) for n in src.names()}, device=device), hf


class Translator:
    """Tokenizer + model + language pair. ``tokenizer`` needs ``encode`` / ``decode`` and a way to turn a
    language code into its token id (``convert_tokens_to_ids`` of HF tokenizers, or ``lang_ids``)."""

    def __init__(self, model, tokenizer, src_lang: str, tgt_lang: str, num_beams: int = 4, lang_ids: Optional[Dict[str, int]] = None):
        self.model, self.tok, self.src_lang, self.tgt_lang, self.num_beams = model, tokenizer, src_lang, tgt_lang, num_beams
        self.lang_ids = lang_ids or {}

    def lang_id(self, code: str) -> int:
        if code in self.lang_ids:
            return self.lang_ids[code]
        conv = getattr(self.tok, "convert_tokens_to_ids", None)
        tid = conv(code) if conv else None
        if tid is None or tid == getattr(self.tok, "unk_token_id", None):
            raise ValueError(f"unknown language code {code!r}")
        return int(tid)

    def translate(self, text: str, src_lang: Optional[str] = None, tgt_lang: Optional[str] = None,
                  max_new_tokens: int = 200) -> Dict[str, Any]:
        src, tgt = self.lang_id(src_lang or self.src_lang), self.lang_id(tgt_lang or self.tgt_lang)
        eos = self.model.cfg.eos_token_id
        out, n_in, n_out = [], 0, 0
        for sent in [s for s in re.split(r"(?<=[.!?。！？])\s+|\n+", text) if s.strip()]:
            ids = [src] + [t for t in self.tok.encode(sent) if t not in (src, eos)] + [eos]
            ids = ids[: self.model.cfg.max_position_embeddings]
            hyp = self.model.translate(ids, tgt, num_beams=self.num_beams, max_new_tokens=max_new_tokens)
            out.append(self.tok.decode(hyp).strip())
            n_in += len(ids)
            n_out += len(hyp)
        return {"text": " ".join(out), "prompt_tokens": n_in, "completion_tokens": n_out}


def create_translation_app(tr: Translator, model_name: str = "nllb"):
    from fastapi import FastAPI, HTTPException
    app = FastAPI(title="metrale-b200 translation")

    def run(text, body):
        if not isinstance(text, str) or not text.strip():
            raise HTTPException(400, "nothing to translate")
        try:
            return tr.translate(text, body.get("src_lang"), body.get("tgt_lang"),
                                int(body.get("max_tokens") or body.get("max_completion_tokens") or 200))
        except ValueError as e:
            raise HTTPException(400, str(e))

    def usage(r):
        return {"prompt_tokens": r["prompt_tokens"], "completion_tokens": r["completion_tokens"],
                "total_tokens": r["prompt_tokens"] + r["completion_tokens"]}

    @app.get("/health")
    def health():
        return {"status": "ok", "model": model_name, "task": "translation", "src_lang": tr.src_lang, "tgt_lang": tr.tgt_lang}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "local"}]}

    @app.post("/v1/completions")
    def completions(body: Dict[str, Any]):
        p = body.get("prompt")
        r = run(p[0] if isinstance(p, list) and p else p, body)
        return {"id": "cmpl-" + uuid.uuid4().hex[:16], "object": "text_completion", "created": int(time.time()),
                "model": model_name, "choices": [{"index": 0, "text": r["text"], "finish_reason": "stop"}], "usage": usage(r)}

    @app.post("/v1/chat/completions")
    def chat(body: Dict[str, Any]):
        from .chat_template import _content_to_text
        users = [m for m in body.get("messages") or [] if m.get("role") == "user"]
        if not users:
            raise HTTPException(400, "no user message to translate")
        r = run(_content_to_text(users[-1].get("content")), body)
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:16], "object": "chat.completion", "created": int(time.time()),
                "model": model_name, "choices": [{"index": 0, "message": {"role": "assistant", "content": r["text"]},
                                                  "finish_reason": "stop"}], "usage": usage(r)}

    return app
