"""Requests with images: the vision tower's embeddings for the prompt's placeholder tokens and the
three-axis rotary index, prepared once at admission and consumed by the runner on every step that holds
the sequence (``ModelRunner._attach_multimodal``)."""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Dict, List, Sequence

import torch


@dataclass
class MultiModalInputs:
    embeds: torch.Tensor                 # [placeholders, hidden] on the engine's device
    row_of_token: Dict[int, int]         # prompt token index -> row of `embeds`
    positions: torch.Tensor              # [3, prompt_len] int64 (host)
    delta: int                           # rotary position of generated token i = i + delta
    digest: str                          # identifies the images in the prefix cache
    grids: List[tuple] = field(default_factory=list)


def expand_placeholders(prompt_ids: Sequence[int], image_token_id: int, counts: Sequence[int]) -> List[int]:
    """A prompt that marks each image with ONE placeholder token -> the prompt with that token repeated
    to the number of embeddings the image yields. A prompt whose runs already have the right lengths is
    returned unchanged."""
    runs, i, n = [], 0, len(prompt_ids)
    while i < n:
        if prompt_ids[i] == image_token_id:
            j = i
            while j < n and prompt_ids[j] == image_token_id:
                j += 1
            runs.append((i, j - i))
            i = j
        else:
            i += 1
    if len(runs) != len(counts):
        raise ValueError(f"the prompt marks {len(runs)} images, the request carries {len(counts)}")
    if all(r[1] == c for r, c in zip(runs, counts)):
        return list(prompt_ids)
    if any(r[1] != 1 for r in runs):
        raise ValueError("image placeholder runs must be one token each or already expanded to the image's size")
    out, last = [], 0
    for (start, _), c in zip(runs, counts):
        out += list(prompt_ids[last:start]) + [image_token_id] * c
        last = start + 1
    return out + list(prompt_ids[last:])


def build_inputs(prompt_ids: Sequence[int], images: Sequence, *, encoder, preprocessor, image_token_id: int,
                 merge: int, device) -> tuple:
    """Returns (expanded prompt ids, MultiModalInputs)."""
    from ..vision.mrope import mrope_positions
    patches, grid = preprocessor(images)
    embeds = encoder(patches, grid).to(torch.bfloat16).to(device)
    grids = [tuple(g) for g in grid.tolist()]
    counts = [t * (h // merge) * (w // merge) for t, h, w in grids]
    ids = expand_placeholders(prompt_ids, image_token_id, counts)
    pos, delta = mrope_positions(ids, image_token_id, grids, merge)
    rows, k = {}, 0
    for i, tok in enumerate(ids):
        if tok == image_token_id:
            rows[i] = k
            k += 1
    if k != embeds.shape[0]:
        raise ValueError(f"{k} placeholder tokens for {embeds.shape[0]} image embeddings")
    digest = hashlib.sha256(patches.numpy().tobytes() + str(grids).encode()).hexdigest()[:32]
    return ids, MultiModalInputs(embeds, rows, pos, delta, digest, grids)
