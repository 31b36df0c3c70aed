"""Record codecs of the KV tier: how one floating-point field of a cached block is stored outside the device pool.

``raw``      the pool's own bytes.
``nvfp4``    e2m1 values, one e4m3 scale per 16 channels, one fp32 scale per row (the checkpoint weight format
             applied to cached rows): K/2 + K/16 + 4 bytes per row of K channels.
``turbo2`` / ``turbo3`` / ``turbo4``
             the row is rotated by a normalised Walsh-Hadamard transform (over the largest power-of-two block that
             divides K), which spreads outliers so that the rotated channels are close to Gaussian with the row's
             rms; each channel is then stored as the index of the nearest Lloyd-Max level of a unit Gaussian
             (4 / 8 / 16 levels), bit-packed, with the rms as one fp32 per row: K * bits / 8 + 4 bytes per row.
             Decoding looks the levels up, scales by the rms and rotates back (the transform is its own inverse).

All of them work on any device with plain tensor ops: they run when a block leaves or re-enters the pool, not in
the attention kernels, whose pools hold bf16 or e4m3.

Reference: the KV cache dtypes of ``crates/cache/src/kv_cache.rs:26-70`` (fp8, nvfp4, turbo2/3/4/8) and the
Walsh-Hadamard + codebook writers of ``kernels/gb10/common/reshape_and_cache_turbo.cu``; there they are device pool
formats read by dedicated attention kernels, here they are codecs of the tier under the prefix cache.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

# Lloyd-Max reproduction levels of a unit Gaussian (positive half; the quantiser is symmetric)
_LEVELS = {
    2: (0.4528, 1.5104),
    3: (0.2451, 0.7560, 1.3439, 2.1520),
    4: (0.1284, 0.3881, 0.6568, 0.9424, 1.2562, 1.6181, 2.0690, 2.7326),
}


def hadamard_block(K: int) -> int:
    """Largest power of two that divides K."""
    return K & -K


def fwht(x: torch.Tensor, block: int) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform over consecutive blocks of the last dimension (self-inverse)."""
    if block < 2:
        return x
    R, K = x.shape
    y = x.reshape(R, K // block, block)
    h = 1
    while h < block:
        y = y.reshape(R, K // block, block // (2 * h), 2, h)
        a, b = y[:, :, :, 0, :], y[:, :, :, 1, :]
        y = torch.stack((a + b, a - b), dim=3)
        h *= 2
    return y.reshape(R, K) * (1.0 / math.sqrt(block))


def _pack_bits(idx: torch.Tensor, bits: int) -> torch.Tensor:
    """idx [R, K] of values < 2**bits -> uint8 [R, K * bits / 8] (little-endian bit order within the row)."""
    R, K = idx.shape
    shifts = torch.arange(bits, device=idx.device)
    b = ((idx.to(torch.int32)[:, :, None] >> shifts) & 1).reshape(R, K * bits // 8, 8)
    w = (1 << torch.arange(8, device=idx.device)).to(torch.int32)
    return (b * w).sum(-1).to(torch.uint8)


def _unpack_bits(packed: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    R = packed.shape[0]
    shifts = torch.arange(8, device=packed.device)
    b = ((packed.to(torch.int32)[:, :, None] >> shifts) & 1).reshape(R, K, bits)
    w = (1 << torch.arange(bits, device=packed.device)).to(torch.int32)
    return (b * w).sum(-1)


class Codec:
    name = "raw"

    def row_bytes(self, K: int, elem: int) -> int:
        return K * elem

    def applies(self, dtype: torch.dtype, K: int) -> bool:
        return False


class Nvfp4Codec(Codec):
    name = "nvfp4"

    def applies(self, dtype, K):
        return dtype in (torch.bfloat16, torch.float16, torch.float32) and K % 16 == 0

    def row_bytes(self, K, elem):
        return K // 2 + K // 16 + 4

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        from ..ops import reference as ref
        q, sf, g = ref.quantize_nvfp4(x.float())
        return torch.cat([q, sf, g.float().contiguous().view(-1, 1).view(torch.uint8).reshape(x.shape[0], 4)], dim=1)

    def decode(self, rec: torch.Tensor, K: int) -> torch.Tensor:
        from ..ops import reference as ref
        q, sf, g = rec[:, :K // 2], rec[:, K // 2:K // 2 + K // 16], rec[:, K // 2 + K // 16:]
        return ref.dequantize_nvfp4(q.contiguous(), sf.contiguous(), g.contiguous().view(torch.float32).reshape(-1))


class TurboCodec(Codec):
    def __init__(self, bits: int):
        if bits not in _LEVELS:
            raise ValueError(f"turbo codec: {bits} bits is not one of {sorted(_LEVELS)}")
        self.bits, self.name = bits, f"turbo{bits}"
        pos = torch.tensor(_LEVELS[bits], dtype=torch.float32)
        self.levels = torch.cat([-pos.flip(0), pos])                      # ascending, 2**bits entries
        self.edges = (self.levels[1:] + self.levels[:-1]) / 2             # nearest-level decision thresholds

    def applies(self, dtype, K):
        return dtype in (torch.bfloat16, torch.float16, torch.float32) and (K * self.bits) % 8 == 0 and K % 8 == 0

    def row_bytes(self, K, elem):
        return K * self.bits // 8 + 4

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        x = fwht(x.float(), hadamard_block(x.shape[1]))
        rms = x.pow(2).mean(dim=1, keepdim=True).sqrt()
        safe = torch.where(rms > 0, rms, torch.ones_like(rms))           # an all-zero row keeps rms = 0 and decodes to zeros
        idx = torch.bucketize((x / safe).contiguous(), self.edges.to(x.device))
        return torch.cat([_pack_bits(idx, self.bits), rms.contiguous().view(torch.uint8).reshape(x.shape[0], 4)], dim=1)

    def decode(self, rec: torch.Tensor, K: int) -> torch.Tensor:
        n = K * self.bits // 8
        idx = _unpack_bits(rec[:, :n].contiguous(), self.bits, K)
        rms = rec[:, n:].contiguous().view(torch.float32).reshape(-1, 1)
        return fwht(self.levels.to(rec.device)[idx] * rms, hadamard_block(K))


def make_codec(name: str) -> Codec:
    if name == "raw":
        return Codec()
    if name == "nvfp4":
        return Nvfp4Codec()
    if name.startswith("turbo") and name[5:].isdigit():
        return TurboCodec(int(name[5:]))
    raise ValueError(f"kv tier codec must be raw | nvfp4 | turbo2 | turbo3 | turbo4, not {name!r}")


def roundtrip(codec: Codec, x: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """(decoded copy of x [R, K], bytes per row): what a trip through the tier does to a field."""
    rec = codec.encode(x)
    return codec.decode(rec, x.shape[1]), rec.shape[1]
