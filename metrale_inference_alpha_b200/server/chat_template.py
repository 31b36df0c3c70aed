"""Chat prompt rendering: the checkpoint's Jinja chat template when present, else ChatML.
Role of ``crates/server/src/tokenizer/chat_render.rs`` (minijinja there, jinja2 here)."""
from __future__ import annotations

import json
from typing import Any, Dict, List, Optional

import jinja2

CHATML = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n{{ m['content'] }}<|im_end|>\n{% endfor %}"
    "{% if tools %}<|im_start|>system\n# Tools\n{{ tools | tojson }}<|im_end|>\n{% endif %}"
    "{% if add_generation_prompt %}<|im_start|>assistant\n{% if enable_thinking %}<think>\n{% endif %}{% endif %}"
)


IMAGE_PLACEHOLDER = "<|vision_start|><|image_pad|><|vision_end|>"
_IMAGE_PARTS = ("image_url", "input_image", "image")


def image_of_part(p) -> Optional[str]:
    """The image a content part carries, as a data: URL (OpenAI ``image_url`` / ``input_image`` parts,
    Anthropic ``image`` blocks with a base64 source), or None for any other part."""
    if not isinstance(p, dict) or p.get("type") not in _IMAGE_PARTS:
        return None
    if p["type"] == "image":
        src = p.get("source") or {}
        if src.get("type") == "base64":
            return f"data:{src.get('media_type', 'image/png')};base64,{src.get('data', '')}"
        return src.get("url")
    u = p.get("image_url")
    return u.get("url") if isinstance(u, dict) else u


def collect_images(messages) -> List[str]:
    """Images of a conversation in the order their placeholders appear in the rendered prompt."""
    out = []
    for m in messages:
        c = m.get("content")
        if isinstance(c, list):
            out += [u for u in (image_of_part(p) for p in c) if u]
    return out


def _content_to_text(content) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    parts = []
    for p in content:                      # OpenAI content parts / Anthropic blocks
        if isinstance(p, str):
            parts.append(p)
        elif p.get("type") in ("text", "input_text", "output_text"):
            parts.append(p.get("text", ""))
        elif p.get("type") in _IMAGE_PARTS:
            parts.append(IMAGE_PLACEHOLDER)
        elif p.get("type") == "tool_result":
            parts.append(_content_to_text(p.get("content")))
        elif p.get("type") == "tool_use":
            parts.append("<tool_call>\n" + json.dumps({"name": p.get("name"), "arguments": p.get("input", {})})
                         + "\n</tool_call>")
    return "".join(parts)


def normalise_messages(messages: List[Dict[str, Any]]) -> List[Dict[str, Any]]:
    out = []
    for m in messages:
        mm = dict(m)
        mm["content"] = _content_to_text(m.get("content"))
        if m.get("tool_calls"):
            calls = "".join("<tool_call>\n" + json.dumps({"name": c["function"]["name"],
                            "arguments": json.loads(c["function"].get("arguments") or "{}")}) + "\n</tool_call>"
                            for c in m["tool_calls"])
            mm["content"] = (mm["content"] + calls) if mm["content"] else calls
        out.append(mm)
    return out


class ChatRenderer:
    def __init__(self, template: Optional[str] = None):
        env = jinja2.Environment(trim_blocks=False, lstrip_blocks=False, keep_trailing_newline=True)
        env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False)
        env.globals["raise_exception"] = self._raise
        self.template = env.from_string(template or CHATML)

    @staticmethod
    def _raise(msg):
        raise jinja2.TemplateError(msg)

    def render(self, messages, tools=None, add_generation_prompt=True, enable_thinking=False, **kwargs) -> str:
        return self.template.render(messages=normalise_messages(messages), tools=tools or None,
                                    add_generation_prompt=add_generation_prompt,
                                    enable_thinking=enable_thinking, **kwargs)
