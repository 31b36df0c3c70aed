"""Multimodal rotary positions: three position axes (time, height, width) per token.

Text tokens advance all three axes together. The placeholder tokens of an image share one time
position and take the (row, column) of their merged patch on the other two axes, offset by the position
where the image starts; the text after an image resumes at one past the largest position used so far.
Generation continues from ``len(tokens) + delta`` on all axes. The rotary kernel consumes the axes
through per-token cos / sin rows gathered section by section (``gather_tables``).

Reference: the multimodal rotary index of the Qwen-VL family (``rope_mrope_interleaved`` kernels in
``kernels/gb10/common``).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def mrope_positions(tokens: Sequence[int], image_token_id: int, grids: Sequence[Tuple[int, int, int]],
                    merge: int = 2) -> Tuple[torch.Tensor, int]:
    """``tokens`` with runs of ``image_token_id`` (one run per image, ``t * (h/merge) * (w/merge)`` long) ->
    (positions [3, len(tokens)] int64, delta) with next position = len(tokens) + delta."""
    pos: List[List[int]] = [[], [], []]
    i, nxt, img = 0, 0, 0
    n = len(tokens)
    while i < n:
        if tokens[i] != image_token_id:
            for a in range(3):
                pos[a].append(nxt)
            nxt += 1
            i += 1
            continue
        if img >= len(grids):
            raise ValueError("more image placeholder runs than images")
        t, h, w = grids[img]
        gh, gw = h // merge, w // merge
        cnt = t * gh * gw
        if list(tokens[i:i + cnt]) != [image_token_id] * cnt:
            raise ValueError(f"image {img}: expected a run of {cnt} placeholder tokens")
        for ti in range(t):
            for r in range(gh):
                for c in range(gw):
                    pos[0].append(nxt + ti)
                    pos[1].append(nxt + r)
                    pos[2].append(nxt + c)
        nxt += max(t, gh, gw)
        i += cnt
        img += 1
    if img != len(grids):
        raise ValueError("fewer image placeholder runs than images")
    return torch.tensor(pos, dtype=torch.int64), nxt - n


def gather_tables(cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor, sections: Sequence[int]):
    """Per-token rotary rows for three-axis positions: frequency i takes its angle from the axis whose
    section it falls in (``sections`` = number of frequencies per axis, summing to rot / 2). ``cos`` /
    ``sin`` [max_pos, rot / 2], ``positions`` [3, T] -> ([T, rot / 2], [T, rot / 2])."""
    half = cos.shape[1]
    if sum(sections) != half:
        raise ValueError(f"mrope sections {list(sections)} must sum to {half}")
    axis = torch.repeat_interleave(torch.arange(3, device=cos.device), torch.tensor(list(sections), device=cos.device))
    idx = positions.to(cos.device)[axis, :].T                                   # [T, half]: the position each frequency uses
    cols = torch.arange(half, device=cos.device)[None, :].expand_as(idx)
    return cos[idx, cols], sin[idx, cols]
