"""Splits generated text into reasoning and answer, incrementally.
Formats: ``<think>...</think>`` (Qwen / DeepSeek-R1 / MiniMax; the prompt may already have
opened the block), ``[THINK]...[/THINK]`` (Mistral), ``<|channel>...<channel|>`` (Gemma).
Role of ``crates/server/src/reasoning_parser/mod.rs:3-16``."""
from __future__ import annotations

from typing import Tuple

FORMATS = {"think": ("<think>", "</think>"), "mistral": ("[THINK]", "[/THINK]"),
           "gemma": ("<|channel>", "<channel|>"), "gemma4": ("<|channel>", "<channel|>")}


class ReasoningParser:
    def __init__(self, fmt: str = "think", starts_open: bool = False):
        self.open_tag, self.close_tag = FORMATS[fmt]
        self.in_reasoning = starts_open
        self.done = False
        self._buf = ""

    def push(self, text: str) -> Tuple[str, str]:
        """Returns (reasoning_delta, content_delta); holds back a possible partial tag."""
        self._buf += text
        r_out, c_out = "", ""
        while self._buf:
            if self.done:
                c_out += self._buf
                self._buf = ""
                break
            tag = self.close_tag if self.in_reasoning else self.open_tag
            i = self._buf.find(tag)
            if i >= 0:
                head = self._buf[:i]
                if self.in_reasoning:
                    r_out += head
                    self.in_reasoning, self.done = False, True
                else:
                    c_out += head
                    self.in_reasoning = True
                self._buf = self._buf[i + len(tag):]
                continue
            # keep a suffix that could be the start of the tag
            keep = 0
            for k in range(min(len(tag) - 1, len(self._buf)), 0, -1):
                if tag.startswith(self._buf[-k:]):
                    keep = k
                    break
            emit = self._buf[:len(self._buf) - keep]
            if self.in_reasoning:
                r_out += emit
            else:
                c_out += emit
                if emit.strip():
                    self.done = not self.in_reasoning and False
            self._buf = self._buf[len(self._buf) - keep:]
            break
        return r_out, c_out

    def flush(self) -> Tuple[str, str]:
        rest, self._buf = self._buf, ""
        return (rest, "") if self.in_reasoning else ("", rest)


def split_reasoning(text: str, fmt: str = "think", starts_open: bool = False) -> Tuple[str, str]:
    p = ReasoningParser(fmt, starts_open)
    r, c = p.push(text)
    r2, c2 = p.flush()
    return r + r2, c + c2
