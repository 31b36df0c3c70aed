"""Prompt-lookup (n-gram) drafter: find the most recent earlier occurrence of the last n
tokens and propose what followed it. Needs no model.
(``crates/speculative/src/ngram.rs:46-70``.)"""
from __future__ import annotations

from typing import List, Sequence


class NgramProposer:
    def __init__(self, max_n: int = 4, min_n: int = 2, window: int = 4096):
        self.max_n, self.min_n, self.window = max_n, min_n, window

    def propose(self, tokens: Sequence[int], k: int) -> List[int]:
        L = len(tokens)
        if k <= 0 or L < self.min_n + 1:
            return []
        lo = max(0, L - self.window)
        for n in range(min(self.max_n, L - 1), self.min_n - 1, -1):
            tail = list(tokens[L - n:])
            for start in range(L - n - 1, lo - 1, -1):      # most recent match first
                if list(tokens[start:start + n]) == tail:
                    cont = list(tokens[start + n:start + n + k])
                    if cont:
                        return cont
        return []


def propose_from_prediction(output: List[int], prediction: List[int], k: int, anchor: int = 3) -> List[int]:
    """Drafts from a caller-supplied predicted output (OpenAI `prediction`): while the output
    follows the prediction, the next k predicted tokens; after a divergence, the continuation of
    the place in the prediction where the last `anchor` output tokens occur that lies closest to
    the current output length (an edit in the middle of a file re-synchronises a few tokens later,
    and repetitive text stays aligned); nothing when there is no such place."""
    n = len(output)
    if k <= 0 or not prediction:
        return []
    if n <= len(prediction) and prediction[:n] == output:
        return list(prediction[n:n + k])
    if n < anchor:
        return []
    tail = output[-anchor:]
    best = -1
    for i in range(len(prediction) - anchor + 1):
        if prediction[i:i + anchor] == tail and (best < 0 or abs(i + anchor - n) <= abs(best + anchor - n)):   # ties: the later place
            best = i
    return list(prediction[best + anchor:best + anchor + k]) if best >= 0 else []
