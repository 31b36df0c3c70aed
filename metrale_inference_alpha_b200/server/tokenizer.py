"""Tokenizer access for the server: a HF ``tokenizer.json`` when the checkpoint ships one,
otherwise a byte-level fallback (ids 0..255 are bytes, 256+ specials) so synthetic models can be
served. Includes the incremental detokeniser used by the SSE streams (holds back incomplete
UTF-8 sequences). Role of ``crates/server/src/tokenizer.rs``."""
from __future__ import annotations

import json
from pathlib import Path
from typing import List, Optional


class ByteTokenizer:
    """ids 0..255 = raw bytes; 256 = <bos>, 257 = <eos>, 258.. = chat markers."""
    SPECIALS = ["<|bos|>", "<|eos|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>",
                "<tool_call>", "</tool_call>", "<|vision_start|>", "<|image_pad|>", "<|vision_end|>"]

    def __init__(self, vocab_size: int = 4096):
        self.vocab_size = vocab_size
        self.bos_token_id, self.eos_token_id = 256, 257
        self._sp = {s: 256 + i for i, s in enumerate(self.SPECIALS)}
        self._inv = {v: k for k, v in self._sp.items()}

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        out: List[int] = [self.bos_token_id] if add_special_tokens else []
        i = 0
        while i < len(text):
            for s, tid in self._sp.items():
                if text.startswith(s, i):
                    out.append(tid)
                    i += len(s)
                    break
            else:
                out.extend(text[i].encode("utf-8"))
                i += 1
        return out

    def token_bytes(self, tid: int) -> bytes:
        if tid < 256:
            return bytes([tid])
        if tid in self._inv:
            return self._inv[tid].encode()
        return b""            # ids beyond the byte range carry no text

    def decode(self, ids: List[int], skip_special_tokens: bool = True) -> str:
        b = b"".join(self.token_bytes(t) for t in ids if not (skip_special_tokens and t in (256, 257)))
        return b.decode("utf-8", errors="replace")


class HfTokenizer:
    def __init__(self, path: Path):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(str(path / "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size()
        cfg = {}
        for name in ("tokenizer_config.json", "generation_config.json", "config.json"):
            f = path / name
            if f.exists():
                cfg.update({k: v for k, v in json.loads(f.read_text()).items() if k not in cfg})
        self.chat_template = cfg.get("chat_template")
        self.eos_token_id = self._tok_id(cfg.get("eos_token"), cfg.get("eos_token_id"))
        self.bos_token_id = self._tok_id(cfg.get("bos_token"), cfg.get("bos_token_id"))

    def _tok_id(self, tok, tid):
        if isinstance(tid, list):
            tid = tid[0]
        if isinstance(tid, int):
            return tid
        if isinstance(tok, dict):
            tok = tok.get("content")
        return self.tk.token_to_id(tok) if tok else None

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids: List[int], skip_special_tokens: bool = True) -> str:
        return self.tk.decode(ids, skip_special_tokens=skip_special_tokens)

    def token_bytes(self, tid: int) -> bytes:
        return self.tk.decode([tid], skip_special_tokens=False).encode()


def load_tokenizer(path: Optional[str], vocab_size: int = 4096):
    if path and (Path(path) / "tokenizer.json").exists():
        return HfTokenizer(Path(path))
    return ByteTokenizer(vocab_size)


class IncrementalDetokenizer:
    """Feeds token ids, returns only text that can no longer change: decodes a sliding window
    and withholds a trailing replacement character (an incomplete multi-byte sequence)."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tk = tokenizer
        self.ids: List[int] = []
        self.prefix_off = 0          # ids[prefix_off:read_off] already emitted as text
        self.read_off = 0
        self.skip = skip_special_tokens

    def push(self, new_ids: List[int]) -> str:
        self.ids.extend(new_ids)
        prefix = self.tk.decode(self.ids[self.prefix_off:self.read_off], self.skip)
        full = self.tk.decode(self.ids[self.prefix_off:], self.skip)
        if full.endswith("�"):
            return ""
        out = full[len(prefix):]
        self.prefix_off = self.read_off
        self.read_off = len(self.ids)
        return out

    def flush(self) -> str:
        prefix = self.tk.decode(self.ids[self.prefix_off:self.read_off], self.skip)
        full = self.tk.decode(self.ids[self.prefix_off:], self.skip)
        self.prefix_off = self.read_off = len(self.ids)
        return full[len(prefix):]
