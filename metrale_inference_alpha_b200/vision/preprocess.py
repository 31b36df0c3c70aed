"""Image preprocessing for the Qwen-VL vision tower: decode, resize to a grid the tower accepts,
normalise, and cut into the flattened patch matrix in merge-group order.

``smart_resize`` keeps the aspect ratio, makes both sides multiples of ``patch * merge`` and keeps the
pixel count inside ``[min_pixels, max_pixels]``. ``patchify`` emits rows of ``C * Tp * P * P`` values
ordered (frame group, merged row, merged column, row in group, column in group), the order the tower's
rotary index and its 2x2 merger assume. Images arrive as uint8 arrays / tensors ``[H, W, 3]``, PIL
images, raw PNG / JPEG bytes or ``data:`` URLs (the form OpenAI-style ``image_url`` parts carry; remote
URLs are refused: the server makes no outbound requests).
"""
from __future__ import annotations

import base64
import io
import math
from dataclasses import dataclass
from typing import List, Sequence, Tuple, Union

import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> Tuple[int, int]:
    if min(height, width) <= 0:
        raise ValueError("image sides must be positive")
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200 is refused")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def decode_image(src) -> torch.Tensor:
    """Any accepted image form -> uint8 tensor [H, W, 3]."""
    if isinstance(src, torch.Tensor):
        t = src
    elif isinstance(src, str):
        if not src.startswith("data:"):
            raise ValueError("only data: URLs are accepted for images (no outbound requests are made)")
        head, _, payload = src.partition(",")
        if ";base64" not in head:
            raise ValueError("image data URLs must be base64")
        return decode_image(base64.b64decode(payload))
    elif isinstance(src, (bytes, bytearray)):
        from PIL import Image
        import numpy as np
        with Image.open(io.BytesIO(bytes(src))) as im:
            t = torch.from_numpy(np.array(im.convert("RGB")))
    else:
        import numpy as np
        arr = np.array(src.convert("RGB")) if hasattr(src, "convert") else np.asarray(src)
        t = torch.from_numpy(arr.copy())
    if t.ndim != 3 or t.shape[-1] != 3:
        raise ValueError(f"expected an [H, W, 3] image, got {tuple(t.shape)}")
    return t.to(torch.uint8)


@dataclass
class ImagePreprocessor:
    patch_size: int = 14
    merge_size: int = 2
    temporal_patch_size: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 14 * 14 * 4 * 1280
    mean: Sequence[float] = CLIP_MEAN
    std: Sequence[float] = CLIP_STD

    def resize_normalize(self, img: torch.Tensor) -> torch.Tensor:
        """uint8 [H, W, 3] -> fp32 [3, H', W'] resized (bicubic, antialiased) and normalised."""
        H, W, _ = img.shape
        h, w = smart_resize(H, W, self.patch_size * self.merge_size, self.min_pixels, self.max_pixels)
        x = img.permute(2, 0, 1).float()[None]
        if (h, w) != (H, W):
            x = F.interpolate(x, size=(h, w), mode="bicubic", antialias=True, align_corners=False).clamp(0, 255).round()
        x = x[0] / 255.0
        mean, std = torch.tensor(self.mean)[:, None, None], torch.tensor(self.std)[:, None, None]
        return (x - mean) / std

    def patchify(self, frames: torch.Tensor) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
        """``frames`` [F, 3, H, W] (one image = one frame, repeated up to the temporal patch) ->
        (patch rows [grid_t * gh * gw, 3 * Tp * P * P], (grid_t, gh, gw))."""
        Tp, P, m = self.temporal_patch_size, self.patch_size, self.merge_size
        if frames.shape[0] % Tp:
            frames = torch.cat([frames, frames[-1:].expand(Tp - frames.shape[0] % Tp, -1, -1, -1)], 0)
        Fr, C, H, W = frames.shape
        gt, gh, gw = Fr // Tp, H // P, W // P
        x = frames.reshape(gt, Tp, C, gh // m, m, P, gw // m, m, P)
        x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)               # frame group, merged row, merged col, in-group row, col, C, Tp, P, P
        return x.reshape(gt * gh * gw, C * Tp * P * P).contiguous(), (gt, gh, gw)

    def __call__(self, images: Sequence) -> Tuple[torch.Tensor, torch.Tensor]:
        """A list of images -> (patch matrix of all images, grid_thw [num_images, 3])."""
        rows, grids = [], []
        for src in images:
            x = self.resize_normalize(decode_image(src))
            p, g = self.patchify(x[None])
            rows.append(p)
            grids.append(g)
        return torch.cat(rows, 0), torch.tensor(grids, dtype=torch.long)

    def num_image_tokens(self, height: int, width: int) -> int:
        """LLM placeholder tokens an image of this size expands to."""
        h, w = smart_resize(height, width, self.patch_size * self.merge_size, self.min_pixels, self.max_pixels)
        return (h // self.patch_size) * (w // self.patch_size) // self.merge_size ** 2
