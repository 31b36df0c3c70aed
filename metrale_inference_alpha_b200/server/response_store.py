"""In-memory store of `/v1/responses` results (bounded LRU) so that a follow-up request can
continue a conversation with `previous_response_id`: the stored input and output messages are
prepended to the new input. Role of the reference's response / conversation stores
(``crates/server/src/stores``)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional


class ResponseStore:
    def __init__(self, capacity: int = 1024):
        self.capacity = capacity
        self._d: "OrderedDict[str, dict]" = OrderedDict()

    def put(self, response_id: str, messages: List[dict], output_text: str, previous: Optional[str] = None) -> None:
        self._d[response_id] = {"messages": list(messages), "output": output_text, "previous": previous}
        self._d.move_to_end(response_id)
        while len(self._d) > self.capacity:
            self._d.popitem(last=False)

    def get(self, response_id: str) -> Optional[dict]:
        r = self._d.get(response_id)
        if r is not None:
            self._d.move_to_end(response_id)
        return r

    def delete(self, response_id: str) -> bool:
        return self._d.pop(response_id, None) is not None

    def thread(self, response_id: str) -> List[dict]:
        """Messages of the whole chain ending at `response_id`, oldest first."""
        chain, seen = [], set()
        rid: Optional[str] = response_id
        while rid and rid not in seen:
            seen.add(rid)
            r = self.get(rid)
            if r is None:
                raise KeyError(rid)
            chain.append(r)
            rid = r["previous"]
        msgs: List[dict] = []
        for r in reversed(chain):
            msgs += r["messages"] + [{"role": "assistant", "content": r["output"]}]
        return msgs

    def __len__(self) -> int:
        return len(self._d)
