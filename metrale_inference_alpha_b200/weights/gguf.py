"""GGUF checkpoints: container parser (v2 / v3: metadata key-values, tensor directory, aligned data
section), host dequantisation of the common block formats (F32, F16, BF16, Q8_0, Q4_0, Q4_K, Q6_K)
to bf16, the llama.cpp -> HF tensor-name mapping, and a ``TensorSource`` over it, so the regular
loader (and its re-quantisation to the serving formats) runs unchanged. A small writer (F32 / F16 /
Q8_0 / Q4_0) exists for tests and for exporting tiny models.

Role of the reference's GGUF support (``crates/model-weights/src/gguf``: container, CPU dequant;
``crates/config`` GGUF metadata -> ModelConfig). The block layouts are those of the public GGUF /
ggml specification.
"""
from __future__ import annotations

import re
import struct
from pathlib import Path
from typing import Any, BinaryIO, Dict, List, Optional, Tuple

import numpy as np
import torch

from ..config.model_config import ModelConfig
from .source import TensorSource

MAGIC = b"GGUF"
# ggml tensor types
F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 0, 1, 2, 3, 6, 7, 8, 9, 10, 11, 12, 13, 14
BF16 = 30
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q4_0: (32, 18), Q4_K: (256, 144), Q6_K: (256, 210)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


# ----------------------------------------------------------------------------- container
def _rd(f: BinaryIO, fmt: str):
    return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]


def _rd_str(f: BinaryIO) -> str:
    n = _rd(f, "<Q")
    return f.read(n).decode("utf-8", errors="replace")


def _rd_value(f: BinaryIO, t: int):
    if t in _SCALAR:
        return _rd(f, _SCALAR[t])
    if t == 8:
        return _rd_str(f)
    if t == 9:
        et, n = _rd(f, "<I"), _rd(f, "<Q")
        if et in _SCALAR:
            sz = struct.calcsize(_SCALAR[et])
            return list(np.frombuffer(f.read(sz * n), dtype=np.dtype(_SCALAR[et][1:]).newbyteorder("<")))
        return [_rd_value(f, et) for _ in range(n)]
    raise ValueError(f"unknown GGUF value type {t}")


class GgufFile:
    def __init__(self, path):
        self.path = Path(path)
        self.meta: Dict[str, Any] = {}
        self.tensors: Dict[str, Tuple[Tuple[int, ...], int, int]] = {}      # name -> (shape, type, offset)
        with open(self.path, "rb") as f:
            if f.read(4) != MAGIC:
                raise ValueError(f"{path}: not a GGUF file")
            self.version = _rd(f, "<I")
            if self.version not in (2, 3):
                raise ValueError(f"{path}: GGUF version {self.version} is not supported")
            n_tensors, n_kv = _rd(f, "<Q"), _rd(f, "<Q")
            for _ in range(n_kv):
                k = _rd_str(f)
                self.meta[k] = _rd_value(f, _rd(f, "<I"))
            for _ in range(n_tensors):
                name = _rd_str(f)
                nd = _rd(f, "<I")
                dims = tuple(_rd(f, "<Q") for _ in range(nd))               # ggml order: fastest first
                typ, off = _rd(f, "<I"), _rd(f, "<Q")
                self.tensors[name] = (tuple(reversed(dims)), typ, off)
            align = int(self.meta.get("general.alignment", 32))
            self.data_start = (f.tell() + align - 1) // align * align

    def nbytes(self, name: str) -> int:
        shape, typ, _ = self.tensors[name]
        if typ not in BLOCK:
            raise NotImplementedError(f"{name}: ggml type {typ} is not supported")
        n = int(np.prod(shape))
        be, bb = BLOCK[typ]
        return n // be * bb

    def read_raw(self, name: str) -> np.ndarray:
        _, _, off = self.tensors[name]
        with open(self.path, "rb") as f:
            f.seek(self.data_start + off)
            return np.frombuffer(f.read(self.nbytes(name)), dtype=np.uint8)

    def dequant(self, name: str) -> torch.Tensor:
        shape, typ, _ = self.tensors[name]
        return dequantize(self.read_raw(name), typ, int(np.prod(shape))).reshape(shape)

    def dequant_device(self, name: str, device) -> torch.Tensor:
        """The tensor as bf16 on `device`. Block-quantised types are uploaded packed and widened
        by the device kernels (ops/csrc/gguf_dequant.cu); other types take the host path."""
        shape, typ, _ = self.tensors[name]
        dev = torch.device(device)
        if dev.type != "cuda" or typ not in (Q8_0, Q4_0, Q4_K, Q6_K):
            return self.dequant(name).to(torch.bfloat16).to(dev)
        from ..ops import _native, _ptr, _stream
        n = int(np.prod(shape))
        raw = torch.from_numpy(self.read_raw(name).copy()).to(dev)
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        _native.check(_native.lib().mb_gguf_dequant(typ, _ptr(raw), n // BLOCK[typ][0], _ptr(out), _stream()),
                      f"gguf_dequant[type {typ}]")
        return out.view(shape)


# ----------------------------------------------------------------------------- block formats
def _f16(b: np.ndarray) -> np.ndarray:
    return b.view(np.float16).astype(np.float32)


def dequantize(raw: np.ndarray, typ: int, n: int) -> torch.Tensor:
    """Raw block bytes -> fp32 tensor of n values."""
    if typ == F32:
        return torch.from_numpy(raw.view(np.float32).copy())
    if typ == F16:
        return torch.from_numpy(raw.view(np.float16).astype(np.float32))
    if typ == BF16:
        return torch.from_numpy(raw.view(np.int16).copy()).view(torch.bfloat16).float()
    if typ == Q8_0:                       # 32 values: f16 d | 32 x i8
        b = raw.reshape(-1, 34)
        d = _f16(b[:, :2].copy())                                # [nb, 1]
        q = b[:, 2:].view(np.int8).astype(np.float32)
        return torch.from_numpy((q * d).reshape(-1)[:n].copy())
    if typ == Q4_0:                       # 32 values: f16 d | 16 bytes; value j = low nibble of byte j, j + 16 = high
        b = raw.reshape(-1, 18)
        d = _f16(b[:, :2].copy())
        qs = b[:, 2:]
        q = np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.float32) - 8.0
        return torch.from_numpy((q * d).reshape(-1)[:n].copy())
    if typ == Q4_K:                       # 256 values: f16 d, f16 dmin | 12 bytes of 6-bit scales / mins | 128 bytes
        b = raw.reshape(-1, 144)
        d, dmin = _f16(b[:, 0:2].copy()), _f16(b[:, 2:4].copy())
        sc, qs = b[:, 4:16].astype(np.int32), b[:, 16:]
        scales, mins = np.zeros((b.shape[0], 8), np.float32), np.zeros((b.shape[0], 8), np.float32)
        for j in range(8):
            if j < 4:
                scales[:, j], mins[:, j] = sc[:, j] & 63, sc[:, j + 4] & 63
            else:
                scales[:, j] = (sc[:, j + 4] & 0x0F) | ((sc[:, j - 4] >> 6) << 4)
                mins[:, j] = (sc[:, j + 4] >> 4) | ((sc[:, j] >> 6) << 4)
        out = np.zeros((b.shape[0], 256), np.float32)
        for g in range(4):                # 64 values per group: low nibbles then high nibbles of 32 bytes
            q = qs[:, g * 32:(g + 1) * 32]
            out[:, g * 64:g * 64 + 32] = d * scales[:, 2 * g:2 * g + 1] * (q & 0x0F) - dmin * mins[:, 2 * g:2 * g + 1]
            out[:, g * 64 + 32:g * 64 + 64] = d * scales[:, 2 * g + 1:2 * g + 2] * (q >> 4) - dmin * mins[:, 2 * g + 1:2 * g + 2]
        return torch.from_numpy(out.reshape(-1)[:n].copy())
    if typ == Q6_K:                       # 256 values: 128 bytes ql | 64 bytes qh | 16 x i8 scales | f16 d
        b = raw.reshape(-1, 210)
        ql, qh = b[:, :128].astype(np.int32), b[:, 128:192].astype(np.int32)
        sc = b[:, 192:208].view(np.int8).astype(np.float32)
        d = _f16(b[:, 208:210].copy())
        out = np.zeros((b.shape[0], 256), np.float32)
        for half in range(2):             # 128 values per half
            l, h = ql[:, half * 64:(half + 1) * 64], qh[:, half * 32:(half + 1) * 32]
            for quarter in range(4):      # 32 values each
                lo = l[:, (quarter & 1) * 32:(quarter & 1) * 32 + 32]
                lo = (lo & 0x0F) if quarter < 2 else (lo >> 4)
                hi = (h >> (2 * quarter)) & 3
                q = (lo | (hi << 4)).astype(np.float32) - 32.0
                base = half * 128 + quarter * 32
                s = np.repeat(sc[:, half * 8 + quarter * 2:half * 8 + quarter * 2 + 2], 16, axis=1)
                out[:, base:base + 32] = d * s * q
        return torch.from_numpy(out.reshape(-1)[:n].copy())
    raise NotImplementedError(f"ggml type {typ} is not supported")


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    b = x.reshape(-1, 32).astype(np.float32)
    d = np.abs(b).max(1, keepdims=True) / 127.0
    q = np.where(d > 0, np.round(b / np.where(d > 0, d, 1)), 0).astype(np.int8)
    return np.concatenate([d.astype(np.float16).view(np.uint8), q.view(np.uint8)], axis=1).reshape(-1)


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    b = x.reshape(-1, 32).astype(np.float32)
    idx = np.abs(b).argmax(1)
    mx = b[np.arange(b.shape[0]), idx][:, None]
    d = mx / -8.0
    q = np.clip(np.round(np.where(d != 0, b / np.where(d != 0, d, 1), 0) + 8.0), 0, 15).astype(np.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    return np.concatenate([d.astype(np.float16).view(np.uint8), packed], axis=1).reshape(-1)


# ----------------------------------------------------------------------------- writer (tests / tiny exports)
def write_gguf(path, meta: Dict[str, Any], tensors: Dict[str, Tuple[torch.Tensor, int]], alignment: int = 32) -> None:
    """tensors[name] = (fp32 tensor, ggml type in {F32, F16, Q8_0, Q4_0})."""
    def w_str(f, s):
        b = s.encode()
        f.write(struct.pack("<Q", len(b)) + b)

    def w_val(f, v):
        if isinstance(v, bool):
            f.write(struct.pack("<I?", 7, v))
        elif isinstance(v, int):
            f.write(struct.pack("<II", 4, v) if 0 <= v < 2 ** 32 else struct.pack("<Iq", 11, v))
        elif isinstance(v, float):
            f.write(struct.pack("<If", 6, v))
        elif isinstance(v, str):
            f.write(struct.pack("<I", 8))
            w_str(f, v)
        else:
            raise TypeError(type(v))
    blobs, infos, off = [], [], 0
    for name, (t, typ) in tensors.items():
        x = t.detach().float().cpu().numpy()
        raw = {F32: lambda a: a.astype(np.float32).view(np.uint8).reshape(-1),
               F16: lambda a: a.astype(np.float16).view(np.uint8).reshape(-1),
               Q8_0: quantize_q8_0, Q4_0: quantize_q4_0}[typ](np.ascontiguousarray(x))
        infos.append((name, tuple(reversed(x.shape)), typ, off))
        blobs.append(raw)
        off += (len(raw) + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IQQ", 3, len(infos), len(meta) + 1))
        w_str(f, "general.alignment")
        w_val(f, alignment)
        for k, v in meta.items():
            w_str(f, k)
            w_val(f, v)
        for name, dims, typ, o in infos:
            w_str(f, name)
            f.write(struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, o))
        f.write(b"\0" * ((f.tell() + alignment - 1) // alignment * alignment - f.tell()))
        for raw in blobs:
            f.write(raw.tobytes())
            f.write(b"\0" * ((len(raw) + alignment - 1) // alignment * alignment - len(raw)))


# ----------------------------------------------------------------------------- names, config, source
_MAP = [(r"^token_embd\.weight$", "model.embed_tokens.weight"), (r"^output_norm\.weight$", "model.norm.weight"),
        (r"^output\.weight$", "lm_head.weight"),
        (r"^blk\.(\d+)\.attn_norm\.weight$", r"model.layers.\1.input_layernorm.weight"),
        (r"^blk\.(\d+)\.ffn_norm\.weight$", r"model.layers.\1.post_attention_layernorm.weight"),
        (r"^blk\.(\d+)\.attn_q_norm\.weight$", r"model.layers.\1.self_attn.q_norm.weight"),
        (r"^blk\.(\d+)\.attn_k_norm\.weight$", r"model.layers.\1.self_attn.k_norm.weight"),
        (r"^blk\.(\d+)\.attn_(q|k|v)\.(weight|bias)$", r"model.layers.\1.self_attn.\2_proj.\3"),
        (r"^blk\.(\d+)\.attn_output\.weight$", r"model.layers.\1.self_attn.o_proj.weight"),
        (r"^blk\.(\d+)\.ffn_(gate|up|down)\.weight$", r"model.layers.\1.mlp.\2_proj.weight")]


def hf_name(gguf_name: str) -> Optional[str]:
    for pat, rep in _MAP:
        if re.match(pat, gguf_name):
            return re.sub(pat, rep, gguf_name)
    return None


def config_from_gguf(g: GgufFile) -> ModelConfig:
    arch = g.meta.get("general.architecture", "llama")
    m = lambda k, d=None: g.meta.get(f"{arch}.{k}", d)
    hidden, heads = int(m("embedding_length")), int(m("attention.head_count"))
    emb = g.tensors["token_embd.weight"][0]
    return ModelConfig(
        name=str(g.meta.get("general.name", g.path.stem)), arch="dense_gqa", vocab_size=int(emb[0]), hidden_size=hidden,
        num_layers=int(m("block_count")), num_heads=heads, num_kv_heads=int(m("attention.head_count_kv", heads)),
        head_dim=int(m("attention.key_length", hidden // heads)), rope_theta=float(m("rope.freq_base", 10000.0)),
        intermediate_size=int(m("feed_forward_length")), rms_eps=float(m("attention.layer_norm_rms_epsilon", 1e-6)),
        max_position=int(m("context_length", 4096)), qk_norm="blk.0.attn_q_norm.weight" in g.tensors,
        tie_embeddings="output.weight" not in g.tensors, weight_format="bf16", kv_dtype="bf16", mtp_layers=0)


class GgufSource(TensorSource):
    """Serves HF-named bf16 tensors out of a GGUF file (dequantised on demand)."""

    def __init__(self, path, cfg: Optional[ModelConfig] = None, device="cpu"):
        self.device = torch.device(device)     # "cuda": block formats are widened on the device
        self.g = GgufFile(path)
        self.cfg = cfg or config_from_gguf(self.g)
        self.arch = self.g.meta.get("general.architecture", "llama")
        self._names = {hf: n for n in self.g.tensors if (hf := hf_name(n))}
        self.quant_config = None

    def has(self, name):
        return name in self._names

    def names(self):
        return self._names.keys()

    def _unpermute(self, w: torch.Tensor, heads: int) -> torch.Tensor:
        # llama-architecture exports interleave the rotary halves of q / k rows; undo it so that the
        # NeoX-style rope of this engine applies
        d = w.shape[0] // heads
        return w.view(heads, d // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)

    def get(self, name):
        w = (self.g.dequant_device(self._names[name], self.device) if self.device.type == "cuda"
             else self.g.dequant(self._names[name]))
        if self.arch == "llama" and name.endswith(("q_proj.weight", "k_proj.weight")):
            w = self._unpermute(w, self.cfg.num_heads if "q_proj" in name else self.cfg.num_kv_heads)
        return w.to(torch.bfloat16)
