"""In-memory conversations (OpenAI Conversations API): an ordered list of items (messages,
function calls and outputs) with metadata, bounded in count and in items per conversation, oldest
conversation evicted first. ``/v1/responses`` reads a conversation as history when the request
names one and appends its input and output to it.

Role of the reference's ``crates/server/src/conversation_store.rs``.
"""
from __future__ import annotations

import threading
import time
import uuid
from collections import OrderedDict
from typing import Dict, List, Optional

MAX_ITEMS_PER_INSERT = 20
MAX_ITEMS_PER_CONVERSATION = 4096
MAX_METADATA_KEYS = 16


class ConversationError(ValueError):
    def __init__(self, message: str, param: Optional[str] = None, code: Optional[str] = None):
        super().__init__(message)
        self.param, self.code = param, code


def check_metadata(md) -> Dict[str, str]:
    md = md or {}
    if not isinstance(md, dict) or len(md) > MAX_METADATA_KEYS:
        raise ConversationError(f"`metadata` holds at most {MAX_METADATA_KEYS} string pairs", "metadata", "metadata_too_large")
    for k, v in md.items():
        if not isinstance(k, str) or not isinstance(v, str) or len(k) > 64 or len(v) > 512:
            raise ConversationError("`metadata` keys (<= 64 chars) and values (<= 512 chars) must be strings", "metadata",
                                    "metadata_invalid")
    return dict(md)


def normalize_item(item: dict) -> dict:
    if not isinstance(item, dict):
        raise ConversationError("conversation items must be objects", "items", "item_invalid")
    t = item.get("type", "message")
    out = dict(item)
    out["type"] = t
    out.setdefault("id", {"message": "msg_", "function_call": "fc_", "function_call_output": "fco_",
                          "reasoning": "rs_"}.get(t, "item_") + uuid.uuid4().hex[:24])
    if t == "message":
        if out.get("role") not in ("user", "assistant", "system", "developer"):
            raise ConversationError("message items need a role of user | assistant | system | developer", "items",
                                    "item_invalid")
        c = out.get("content")
        if isinstance(c, str):
            kind = "output_text" if out["role"] == "assistant" else "input_text"
            out["content"] = [{"type": kind, "text": c}]
        out.setdefault("status", "completed")
    return out


def item_to_message(item: dict) -> Optional[dict]:
    """Chat message an item contributes to a prompt (None for items that carry no text)."""
    t = item.get("type")
    if t == "message":
        parts = item.get("content") or []
        text = "".join(p.get("text", "") for p in parts if isinstance(p, dict)) if isinstance(parts, list) else str(parts)
        role = "system" if item["role"] == "developer" else item["role"]
        return {"role": role, "content": text}
    if t == "function_call":
        return {"role": "assistant", "content": None,
                "tool_calls": [{"id": item.get("call_id", item["id"]), "type": "function",
                                "function": {"name": item.get("name", ""), "arguments": item.get("arguments", "{}")}}]}
    if t == "function_call_output":
        return {"role": "tool", "tool_call_id": item.get("call_id", ""), "content": str(item.get("output", ""))}
    return None


class ConversationStore:
    def __init__(self, capacity: int = 1024):
        self.capacity = capacity
        self._d: "OrderedDict[str, dict]" = OrderedDict()
        self._lock = threading.Lock()

    def create(self, items: Optional[List[dict]] = None, metadata=None) -> dict:
        items = items or []
        if len(items) > MAX_ITEMS_PER_INSERT:
            raise ConversationError(f"`items` exceeds per-call cap of {MAX_ITEMS_PER_INSERT} (got {len(items)}).", "items",
                                    "items_too_many")
        conv = {"id": "conv_" + uuid.uuid4().hex[:24], "object": "conversation", "created_at": int(time.time()),
                "metadata": check_metadata(metadata), "items": [normalize_item(i) for i in items]}
        with self._lock:
            self._d[conv["id"]] = conv
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)
        return conv

    def get(self, cid: str) -> dict:
        with self._lock:
            c = self._d.get(cid)
            if c is None:
                raise KeyError(cid)
            self._d.move_to_end(cid)
            return c

    def update(self, cid: str, metadata) -> dict:
        c = self.get(cid)
        c["metadata"] = check_metadata(metadata)
        return c

    def delete(self, cid: str) -> bool:
        with self._lock:
            return self._d.pop(cid, None) is not None

    def add_items(self, cid: str, items: List[dict]) -> List[dict]:
        if len(items) > MAX_ITEMS_PER_INSERT:
            raise ConversationError(f"`items` exceeds per-call cap of {MAX_ITEMS_PER_INSERT} (got {len(items)}).", "items",
                                    "items_too_many")
        c = self.get(cid)
        if len(c["items"]) + len(items) > MAX_ITEMS_PER_CONVERSATION:
            raise ConversationError(f"a conversation holds at most {MAX_ITEMS_PER_CONVERSATION} items", "items",
                                    "conversation_full")
        new = [normalize_item(i) for i in items]
        c["items"] += new
        return new

    def list_items(self, cid: str, limit: int = 20, after: Optional[str] = None, order: str = "desc") -> dict:
        items = list(self.get(cid)["items"])
        if order == "desc":
            items.reverse()
        if after:
            ids = [i["id"] for i in items]
            if after not in ids:
                raise ConversationError(f"unknown item {after!r}", "after", "item_not_found")
            items = items[ids.index(after) + 1:]
        limit = max(1, min(int(limit), 100))
        page = items[:limit]
        return {"object": "list", "data": page, "first_id": page[0]["id"] if page else None,
                "last_id": page[-1]["id"] if page else None, "has_more": len(items) > limit}

    def get_item(self, cid: str, item_id: str) -> dict:
        for i in self.get(cid)["items"]:
            if i["id"] == item_id:
                return i
        raise KeyError(item_id)

    def delete_item(self, cid: str, item_id: str) -> dict:
        c = self.get(cid)
        n = len(c["items"])
        c["items"] = [i for i in c["items"] if i["id"] != item_id]
        if len(c["items"]) == n:
            raise KeyError(item_id)
        return c

    def messages(self, cid: str) -> List[dict]:
        return [m for m in (item_to_message(i) for i in self.get(cid)["items"]) if m is not None]

    @staticmethod
    def public(conv: dict) -> dict:
        return {k: conv[k] for k in ("id", "object", "created_at", "metadata")}

    def __len__(self) -> int:
        return len(self._d)
