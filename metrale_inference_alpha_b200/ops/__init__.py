"""Tensor-level op API of the engine.

Every function takes torch tensors. CUDA tensors go to the hand-written sm_100a kernels in
``libmetrale_b200.so`` (and raise if the library is missing: no silent fallback on a GPU box);
CPU tensors go to the fp32 restatement in ``reference.py``, which is also the test oracle.
Both paths implement the same quantised arithmetic (same e4m3 / e2m1 rounding, same scale
granularity), so CPU and GPU agree to accumulation-order noise.
"""
from __future__ import annotations

import os

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _native, reference as ref

KIND = {"bf16": 0, "fp8_row": 1, "nvfp4": 2, "fp8_block": 3}
NATIVE_ACT_FOR_WEIGHT = {"bf16": "bf16", "fp8_row": "fp8_row", "fp8_block": "fp8_g128", "nvfp4": "nvfp4"}
# the activation encoding each weight format is fed with; `set_activation_precision` rewrites it in place
ACT_FOR_WEIGHT = dict(NATIVE_ACT_FOR_WEIGHT)
IN_COPY, IN_RMSNORM, IN_SILU_MUL, IN_RELU2, IN_SIGMOID_GATE, IN_GATED_RMSNORM = range(6)
OUT_MODE = {"bf16": 0, "fp8_row": 1, "fp8_g128": 2, "nvfp4": 3}

launch_count = 0  # kernels launched through this module (bench.py reports it)
# kernel-selection bits of the GEMM launcher (csrc/gemm_args.h)
GEMM_ONE_TILE_PER_CTA, GEMM_DECODE_TILE_ORDER, GEMM_PERSISTENT_PREFILL, GEMM_DSMEM_SPLITK = 16, 64, 128, 256
# prefill GEMMs (several 128-token tiles) also run on the persistent kernel (NVFP4 prefill GEMMs
# measure 1.5x faster there; METRALE_PERSISTENT_PREFILL=0 keeps one tile per CTA)
_PERSIST_PREFILL = GEMM_PERSISTENT_PREFILL if os.environ.get("METRALE_PERSISTENT_PREFILL", "1") != "0" else 0
GEMM_GROUPED_ONE_CTA = 512
_GROUPED_CTAS = GEMM_GROUPED_ONE_CTA if os.environ.get("METRALE_GROUPED_CTAS", "2") == "1" else 0


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device address for a kernel argument. Every caller is a CUDA launch, so a host tensor here
    is a wiring error (it would fault on the device): refuse it on the host instead."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"CUDA kernel argument lives on {t.device} (shape {tuple(t.shape)}, {t.dtype})")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _Runtime:
    """Per-device scratch shared by all launches: split-K / split-KV workspace, the status
    word kernels report bounded-wait timeouts and bounds violations through, SM count."""

    _inst = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.ws_bytes = 96 << 20
        from ..utils.alloc_ledger import ledger
        self.ws = ledger().alloc(self.ws_bytes, torch.uint8, device, "gemm workspace")
        self.attn_ws = ledger().alloc(32 << 20, torch.uint8, device, "attention workspace")
        self.status = ledger().alloc(4, torch.int32, device, "status word")

    @classmethod
    def get(cls, device) -> "_Runtime":
        device = torch.device(device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in cls._inst:
            cls._inst[idx] = _Runtime(torch.device("cuda", idx))
        return cls._inst[idx]

    def ensure_attn_ws(self, nbytes: int):
        if nbytes > self.attn_ws.numel():
            from ..utils.alloc_ledger import ledger
            self.attn_ws = ledger().alloc(int(nbytes * 1.25), torch.uint8, self.device, "attention workspace")


def runtime(device) -> _Runtime:
    return _Runtime.get(device)


def check_status(device) -> int:
    """Read (and clear) the device status word; raises KernelError if a kernel reported a
    timed-out wait or an out-of-range index."""
    rt = runtime(device)
    code = int(rt.status[0].item())
    if code:
        rt.status.zero_()
        raise _native.KernelError(f"device status 0x{code:x} "
                                  f"({'bounds' if code == 0x500 else 'bounded wait expired'})")
    return code


# ----------------------------------------------------------------------------- containers
@dataclass
class QuantWeight:
    """One linear layer's weight in its serving format.

    fmt        data                scale
    bf16       bf16 [N, K]         -
    fp8_row    u8   [N, K]         fp32 [N]
    fp8_block  u8   [N, K]         fp32 [ceil(N/128), ceil(K/128)]
    nvfp4      u8   [N, K/2]       u8 e4m3 [N, K/16] (+ tiled copy on CUDA), gscale fp32
    """
    fmt: str
    N: int
    K: int
    data: torch.Tensor
    scale: Optional[torch.Tensor] = None
    gscale: float = 1.0
    row_gscale: Optional[torch.Tensor] = None   # nvfp4: per-row global scale (fused q|k|v, gate|up)
    sf_tiled: Optional[torch.Tensor] = None
    sf_k64: int = 0
    _deq: Optional[torch.Tensor] = None

    def dequant(self) -> torch.Tensor:
        if self._deq is not None:
            return self._deq
        if self.fmt == "bf16":
            d = self.data.float()
        elif self.fmt == "fp8_row":
            d = ref.from_e4m3(self.data) * self.scale.float()[:, None]
        elif self.fmt == "fp8_block":
            d = ref.dequantize_fp8_block128(self.data, self.scale.float())
        else:
            d = ref.dequantize_nvfp4(self.data, self.scale, self.gscale)
            if self.row_gscale is not None:
                d = d * self.row_gscale.float()[:, None]
        if not self.data.is_cuda:
            self._deq = d
        return d

    def dequant64(self) -> torch.Tensor:
        d = getattr(self, "_deq64", None)
        if d is None:
            d = self.dequant().double()
            if not self.data.is_cuda:
                self._deq64 = d
        return d

    def to(self, device) -> "QuantWeight":
        w = QuantWeight(self.fmt, self.N, self.K, self.data.to(device),
                        None if self.scale is None else self.scale.to(device), self.gscale,
                        None if self.row_gscale is None else self.row_gscale.to(device))
        if w.fmt == "nvfp4" and w.data.is_cuda:
            w.prepare_cuda()
        return w

    def prepare_cuda(self):
        """Build the tiled scale-factor copy tcgen05.cp consumes (done once at load)."""
        kblocks = self.K // 16
        kb_stage = (self.K + 255) // 256
        self.sf_k64 = kb_stage * 4
        nb = (self.N + 127) // 128
        self.sf_tiled = torch.zeros(nb * self.sf_k64 * 512, dtype=torch.uint8, device=self.data.device)
        rc = _native.lib().mb_sf_repack(_ptr(self.scale), _ptr(self.sf_tiled), self.N, kblocks,
                                        self.sf_k64, _stream())
        _native.check(rc, "sf_repack")
        _count()

    def nbytes(self) -> int:
        n = self.data.numel() * self.data.element_size()
        if self.scale is not None:
            n += self.scale.numel() * self.scale.element_size()
        return n


def make_weight(w: torch.Tensor, fmt: str) -> QuantWeight:
    """Quantise a float weight [N, K] into serving format `fmt` (synthetic checkpoints, tests,
    and runtime quantisation of bf16 checkpoints)."""
    N, K = w.shape
    if fmt == "bf16":
        return QuantWeight("bf16", N, K, w.to(torch.bfloat16).contiguous())
    if fmt == "fp8_row":
        q, s = ref.quantize_fp8_rowwise(w)
        return QuantWeight("fp8_row", N, K, q, s)
    if fmt == "fp8_block":
        q, s = ref.quantize_fp8_block128(w)
        return QuantWeight("fp8_block", N, K, q, s)
    if fmt == "nvfp4":
        q, sf, g = ref.quantize_nvfp4(w, per_row_global=False)
        return QuantWeight("nvfp4", N, K, q, sf, float(g))
    raise ValueError(fmt)


@dataclass
class Act:
    """An activation matrix [M, K] in the encoding its consumer GEMM wants."""
    fmt: str
    M: int
    K: int
    data: torch.Tensor                      # bf16 [M,K] | u8 [M,K] | u8 [M,K/2]; CPU: fp32 dequantised
    scale: Optional[torch.Tensor] = None    # fp8_row / nvfp4: [M]; fp8_g128: [K/128, ld]
    sf: Optional[torch.Tensor] = None       # nvfp4 tiled scale factors (CUDA)
    sf_k64: int = 0
    bf16: Optional[torch.Tensor] = None     # extra bf16 copy when requested


_SF_ZERO: dict = {}


def _sf_buffer(dev, M: int, K: int):
    """Tiled scale-factor buffer of an NVFP4 activation [M, K] and its row length in 64-channel
    groups. When K fills whole 256-channel stages every byte is written by the producing kernel
    (fresh memory); otherwise the padding groups must read as zero, and a small ring of
    persistent pre-zeroed buffers per shape is used instead of a memset per call (a producer's
    buffer is consumed by the GEMM right behind it, long before the ring comes round)."""
    sf_k64 = ((K + 255) // 256) * 4
    n = ((M + 127) // 128) * sf_k64 * 512
    if K % 256 == 0:
        return torch.empty(n, dtype=torch.uint8, device=dev), sf_k64
    key = (str(dev), (M + 127) // 128, K)
    ring = _SF_ZERO.get(key)
    if ring is None:
        if torch.cuda.is_current_stream_capturing():        # first use inside a capture: pay the memset once
            return torch.zeros(n, dtype=torch.uint8, device=dev), sf_k64
        ring = _SF_ZERO[key] = [[torch.zeros(n, dtype=torch.uint8, device=dev) for _ in range(4)], 0]
    ring[1] = (ring[1] + 1) % len(ring[0])
    return ring[0][ring[1]], sf_k64


def _count(n: int = 1):
    global launch_count
    launch_count += n


# ----------------------------------------------------------------------------- row ops
def row_op(x: torch.Tensor, out_fmt: str = "bf16", mode: int = IN_COPY, *, K: Optional[int] = None,
           residual=None, write_residual: bool = False, w=None, plus_one: bool = False,
           eps: float = 1e-6, gate=None, head_dim: int = 0, gate_head_stride: int = 0,
           gate_head_off: int = 0, group: int = 0, also_bf16: bool = False, static_scale: float = 0.0,
           scale_pad: int = 0, row_index: Optional[torch.Tensor] = None):
    """Fused producer: builds y = recipe(x) per row and encodes it as `out_fmt`. `static_scale`
    (nvfp4 only): calibrated global scale used instead of the row's amax / (6 * 448).
    `scale_pad` (fp8_g128): extra token columns in the per-group scale matrix (grouped expert GEMMs
    read whole row tiles past the last row). `row_index` (CUDA): int32 list of the rows to work on
    (negative entries are skipped); the other rows' outputs stay unwritten (an expert-sorted layout with
    aligned tiles is mostly padding). Returns (Act,
    residual_out or None). x is bf16 (or fp32 for IN_GATED_RMSNORM inputs)."""
    M = x.shape[0]
    if K is None:
        K = x.shape[1] // 2 if mode == IN_SILU_MUL else x.shape[1]
    if not x.is_cuda:
        return _row_op_ref(x, out_fmt, mode, K, residual, write_residual, w, plus_one, eps, gate,
                           head_dim, gate_head_stride, gate_head_off, group, also_bf16, static_scale)
    L = _native.lib()
    dev = x.device
    a = _native.RowArgs()
    a.static_gs = float(static_scale) if out_fmt == "nvfp4" else 0.0
    a.row_index = _ptr(row_index)
    a.M, a.K, a.in_mode, a.out_mode = (M if row_index is None else row_index.numel()), K, mode, OUT_MODE[out_fmt]
    if x.dtype == torch.float32:
        a.xf32 = _ptr(x)
    else:
        assert x.dtype == torch.bfloat16
        a.x = _ptr(x)
    a.x_ld = x.stride(0)
    res_out = None
    if residual is not None:
        a.residual = _ptr(residual)
    if write_residual:
        res_out = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        a.residual_out = _ptr(res_out)
    a.w = _ptr(w)
    a.w_plus_one = int(plus_one)
    a.eps = eps
    if gate is not None:
        a.gate = _ptr(gate)
        a.gate_ld = gate.stride(0)
    a.head_dim, a.gate_head_stride, a.gate_head_off, a.group = head_dim, gate_head_stride, gate_head_off, group
    act = Act(out_fmt, M, K, None)
    if out_fmt == "bf16":
        act.data = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        a.out_ld = K
    elif out_fmt == "fp8_row":
        act.data = torch.empty(M, K, dtype=torch.uint8, device=dev)
        act.scale = torch.empty(M, dtype=torch.float32, device=dev)
        a.out_ld = K
    elif out_fmt == "fp8_g128":
        ld = ((M + scale_pad + 63) // 64) * 64
        act.data = torch.empty(M, K, dtype=torch.uint8, device=dev)
        # columns past M only scale token rows past M, whose outputs are never stored
        act.scale = torch.empty((K + 127) // 128, ld, dtype=torch.float32, device=dev)
        a.out_ld = K
        a.scale_ld = ld
    else:
        act.data = torch.empty(M, K // 2, dtype=torch.uint8, device=dev)
        act.scale = torch.empty(M, dtype=torch.float32, device=dev)
        act.sf, act.sf_k64 = _sf_buffer(dev, M, K)
        a.out_ld = K // 2
        a.sf = _ptr(act.sf)
        a.sf_k64 = act.sf_k64
    a.out = _ptr(act.data)
    a.scale = _ptr(act.scale)
    if also_bf16 and out_fmt != "bf16":
        act.bf16 = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        a.out_bf16 = _ptr(act.bf16)
        a.out_bf16_ld = K
    elif out_fmt == "bf16":
        act.bf16 = act.data
    _native.check(L.mb_row_op(C.byref(a), _stream()), "row_op")
    _count()
    return act, res_out


def _row_op_ref(x, out_fmt, mode, K, residual, write_residual, w, plus_one, eps, gate, head_dim,
                gate_head_stride, gate_head_off, group, also_bf16, static_scale=0.0):
    xf = x.float()
    res_out = None
    if mode == IN_RMSNORM:
        h = xf
        if residual is not None:
            h = ref.bf16_round(h + residual.float())
        if write_residual:
            res_out = h.to(torch.bfloat16)
        y = ref.rms_norm(h, w if w is not None else torch.ones(K), eps, plus_one)
    elif mode == IN_GATED_RMSNORM:
        y = ref.gated_rms_norm(xf, gate, w if w is not None else torch.ones(K), eps, group)
    elif mode == IN_SILU_MUL:
        y = ref.silu_mul(xf[:, :2 * K])
    elif mode == IN_RELU2:
        y = ref.relu2(xf)
    elif mode == IN_SIGMOID_GATE:
        H = K // head_dim
        g = torch.stack([gate[:, h * gate_head_stride + gate_head_off:
                              h * gate_head_stride + gate_head_off + head_dim] for h in range(H)], 1)
        y = xf * torch.sigmoid(g.float().reshape(x.shape[0], K))
    else:
        y = xf[:, :K]
    act = encode_act_ref(y, out_fmt, static_scale)
    if also_bf16 or out_fmt == "bf16":
        act.bf16 = y.to(torch.bfloat16)
    return act, res_out


def encode_act_ref(y: torch.Tensor, fmt: str, static_scale: float = 0.0) -> Act:
    """CPU encoding: quantise exactly like the kernels, then keep the dequantised fp32 matrix."""
    M, K = y.shape
    if fmt == "bf16":
        d = ref.bf16_round(y)
    elif fmt == "fp8_row":
        q, s = ref.quantize_fp8_rowwise(y)
        d = ref.from_e4m3(q) * s[:, None]
    elif fmt == "fp8_g128":
        q, s = ref.quantize_fp8_group128(y)
        d = ref.from_e4m3(q) * s.t().repeat_interleave(128, 1)[:, :K]
    else:
        q, sf, g = ref.quantize_nvfp4(y, per_row_global=True, static_scale=static_scale)
        d = ref.dequantize_nvfp4(q, sf, g)
    return Act(fmt, M, K, d)


def quantize_act(x: torch.Tensor, fmt: str, static_scale: float = 0.0) -> Act:
    return row_op(x, fmt, IN_COPY, static_scale=static_scale)[0]


# ----------------------------------------------------------------------------- linear
def set_activation_precision(mode: str) -> None:
    """"native": activations are quantised to the weight's own format (W4A4 / W8A8, the tensor-core
    block-scaled GEMMs). "a16": activations stay bf16 and only the weights are low precision
    (W4A16 / W8A16, `_linear_a16`); the accuracy option for checkpoints whose activations have
    outliers that 4- or 8-bit rows cannot hold. Process-wide. Expert GEMMs keep the native format."""
    assert mode in ("native", "a16"), mode
    for k, v in NATIVE_ACT_FOR_WEIGHT.items():
        ACT_FOR_WEIGHT[k] = v if mode == "native" else "bf16"


_A16_GEMV_MAX_M = 32           # up to this many rows: passes of the streaming kernel, 8 rows each
_A16_WS_BYTES = 256 << 20      # bf16 staging band for the tensor-core path


def _linear_a16(act: Act, w: QuantWeight, residual, swiglu: bool, out_f32: bool, out):
    """bf16 activations x quantised weight. M <= 32: the streaming kernel reads the packed weight
    once per 8 rows. Larger M: row bands of the weight are widened to bf16 (at most 256 MB at a
    time) and go through the bf16 tensor-core GEMM, one band per launch pair."""
    M, N, K, dev = act.M, w.N, w.K, act.data.device
    n_out = N // 2 if swiglu else N
    if out is None:
        out = torch.empty(M, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
    L = _native.lib()
    a = _native.A16Args()
    a.kind, a.N, a.K, a.ldx, a.swiglu = KIND[w.fmt], N, K, act.data.stride(0), int(swiglu)
    a.W, a.scale, a.row_gscale, a.gscale = _ptr(w.data), _ptr(w.scale), _ptr(w.row_gscale), float(w.gscale)
    a.scale_ld = w.scale.stride(0) if w.fmt == "fp8_block" else 0
    if M <= _A16_GEMV_MAX_M:
        a.ldo = out.stride(0)
        for m0 in range(0, M, 8):
            a.M = min(8, M - m0)
            a.x = act.data.data_ptr() + m0 * act.data.stride(0) * 2
            a.residual = None if residual is None else residual.data_ptr() + m0 * residual.stride(0) * 2
            assert residual is None or residual.stride(0) == out.stride(0)
            o = out.data_ptr() + m0 * out.stride(0) * out.element_size()
            a.out, a.out_f32 = (None, o) if out_f32 else (o, None)
            _native.check(L.mb_a16_gemv(C.byref(a), _stream()), f"a16_gemv[{w.fmt} M={M} N={N} K={K}]")
            _count()
        return out
    if swiglu and out_f32:                                 # the tensor-core SwiGLU epilogue writes bf16
        y = _linear_a16(act, w, residual, True, False, None)
        out.copy_(y)
        return out
    band = max(256, min(N, (_A16_WS_BYTES // (2 * K)) // 256 * 256))
    rt = runtime(dev)
    if getattr(rt, "a16_ws", None) is None or rt.a16_ws.numel() < band * K:
        rt.a16_ws = torch.empty(band * K, dtype=torch.bfloat16, device=dev)
    for n_lo in range(0, N, band):
        rows = min(band, N - n_lo)
        wb = rt.a16_ws[:rows * K].view(rows, K)
        a.n_lo, a.rows, a.out = n_lo, rows, _ptr(wb)
        _native.check(L.mb_a16_dequant(C.byref(a), _stream()), f"a16_dequant[{w.fmt} N={N} K={K}]")
        _count()
        lo, hi = (n_lo // 2, (n_lo + rows) // 2) if swiglu else (n_lo, n_lo + rows)
        linear(act, QuantWeight("bf16", rows, K, wb), residual=None if residual is None else residual[:, lo:hi],
               swiglu=swiglu, out_f32=out_f32, out=out[:, lo:hi])
    return out


def linear(act: Act, w: QuantWeight, *, residual: Optional[torch.Tensor] = None,
           swiglu: bool = False, out_f32: bool = False, out: Optional[torch.Tensor] = None,
           force_tn: int = 0, force_splits: int = 0, one_tile_per_cta: bool = False, decode_tile_order: bool = False,
           dsmem_splitk: bool = False, grouped=None, no_cluster: bool = False, quant_out: float = 0.0):
    """out[m, n] = sum_k act[m, k] * w[n, k] (+ residual); with `swiglu`, w holds gate/up rows
    interleaved (2j, 2j+1) and the result is silu(gate) * up of width N/2. `quant_out` > 0 (with
    `swiglu`): return the result as an NVFP4 `Act` quantised with that calibrated global scale --
    inside the GEMM epilogue when the persistent kernel serves the shape, else by a row kernel.
    `one_tile_per_cta` keeps the shape off the persistent kernel and `decode_tile_order` keeps
    prefill-sized GEMMs on the decode launch order; `dsmem_splitk` makes a split-K cluster exchange
    its partial tiles over distributed shared memory instead of the L2-resident workspace (all
    three for A/B comparisons and tests)."""
    assert act.K == w.K, (act.K, w.K)
    a16 = act.fmt == "bf16" and w.fmt != "bf16"
    assert a16 or act.fmt == NATIVE_ACT_FOR_WEIGHT[w.fmt], (act.fmt, w.fmt)
    M, N = act.M, w.N
    if a16 and act.data.is_cuda:
        assert grouped is None, "expert GEMMs take activations in the weight's own format"
        y = _linear_a16(act, w, residual, swiglu, out_f32 or quant_out > 0.0, out)
        return quantize_act(y, "nvfp4", static_scale=quant_out) if quant_out > 0.0 else y
    if quant_out > 0.0:
        assert swiglu and residual is None and not out_f32 and grouped is None
        fused = (act.data.is_cuda and M <= 128 and (N + 127) // 128 > runtime(act.data.device).sm_count
                 and w.fmt in ("nvfp4", "fp8_row", "bf16") and (N // 2) % 256 == 0 and not one_tile_per_cta)
        if not fused:
            y = linear(act, w, swiglu=True, out_f32=not act.data.is_cuda, force_tn=force_tn, force_splits=force_splits,
                       one_tile_per_cta=one_tile_per_cta)
            return quantize_act(y, "nvfp4", static_scale=quant_out)
    if not act.data.is_cuda:
        # fp64 accumulation: a row's result must not depend on how many other rows share the call
        # (fp32 BLAS picks different blockings for different M, and a random-weight test model has
        # near-ties everywhere), so that batch-invariance tests on the CPU path are exact
        y = (act.data.double() @ w.dequant64().t()).float()
        if swiglu:
            y = torch.nn.functional.silu(y[:, 0::2]) * y[:, 1::2]
        if residual is not None:
            y = y + residual.float()
        return y if out_f32 else y.to(torch.bfloat16)
    L = _native.lib()
    rt = runtime(act.data.device)
    n_out = N // 2 if swiglu else N
    if grouped is not None:
        n_out = grouped[3] // 2 if swiglu else grouped[3]
    if out is None and quant_out <= 0.0:
        out = torch.empty(M, n_out, dtype=torch.float32 if out_f32 else torch.bfloat16,
                          device=act.data.device)
    a = _native.GemmArgs()
    a.kind, a.M, a.N, a.K, a.ldo = KIND[w.fmt], M, N, w.K, (out.stride(0) if out is not None else n_out)
    a.W, a.X, a.out = _ptr(w.data), _ptr(act.data), _ptr(out)
    a.residual = _ptr(residual)
    a.alpha = 1.0
    if w.fmt == "fp8_row":
        a.w_scale, a.a_scale = _ptr(w.scale), _ptr(act.scale)
    elif w.fmt == "fp8_block":
        a.w_scale, a.a_scale, a.a_ld = _ptr(w.scale), _ptr(act.scale), act.scale.stride(0)
    elif w.fmt == "nvfp4":
        if w.sf_tiled is None:
            w.prepare_cuda()
        a.sfa, a.sfb, a.sf_k64 = _ptr(w.sf_tiled), _ptr(act.sf), w.sf_k64
        assert act.sf_k64 == w.sf_k64
        a.a_scale = _ptr(act.scale)
        a.w_scale = _ptr(w.row_gscale)
        a.alpha = w.gscale
    a.epilogue, a.out_f32 = int(swiglu), int(out_f32)
    a.ws, a.ws_bytes, a.status = _ptr(rt.ws), rt.ws_bytes, _ptr(rt.status)
    a.force_tn, a.force_splits, a.sm_count = force_tn, force_splits, rt.sm_count
    a.flags = (_PERSIST_PREFILL | _GROUPED_CTAS | (GEMM_ONE_TILE_PER_CTA if one_tile_per_cta else 0)
               | (GEMM_DECODE_TILE_ORDER if decode_tile_order else 0) | (GEMM_DSMEM_SPLITK if dsmem_splitk else 0))
    a.no_cluster = int(no_cluster)
    qact = None
    if quant_out > 0.0:
        Kq, dev = N // 2, act.data.device
        qact = Act("nvfp4", M, Kq, torch.empty(M, Kq // 2, dtype=torch.uint8, device=dev))
        qact.sf_k64 = Kq // 64
        qact.sf = torch.empty(((M + 127) // 128) * qact.sf_k64 * 512, dtype=torch.uint8, device=dev)
        qact.scale = static_scale_vec(dev, quant_out, M)
        a.out = _ptr(qact.data)                              # the bf16 output does not exist in this mode
        a.outq, a.ldq, a.outq_sf, a.outq_sf_k64, a.outq_gs = _ptr(qact.data), Kq // 2, _ptr(qact.sf), qact.sf_k64, quant_out
    if grouped is not None:
        # (tile_expert, tile_row0, tile_nrows, n_per_expert, max_tiles, tile_rows)
        a.tile_expert, a.tile_row0, a.tile_nrows = _ptr(grouped[0]), _ptr(grouped[1]), _ptr(grouped[2])
        a.n_per_expert, a.max_tiles, a.force_tn = grouped[3], grouped[4], grouped[5]
    _native.check(L.mb_gemm(C.byref(a), _stream()), f"gemm[{w.fmt} M={M} N={N} K={w.K}]")
    _count()
    return qact if qact is not None else out


_SCALE_VECS: dict = {}


def static_scale_vec(device, gs: float, M: int) -> torch.Tensor:
    """[M] fp32 filled with a static activation scale (the per-token scale array the W4A4 GEMM
    epilogue reads). Vectors are created once per (device, scale), outside any stream capture:
    the engine calls this at calibration time; a miss during capture allocates without caching."""
    key = (str(device), float(gs))
    t = _SCALE_VECS.get(key)
    if t is None or t.numel() < M:
        n = max(256, M)
        t = torch.full((n,), float(gs), dtype=torch.float32, device=device)
        if torch.device(device).type == "cuda" and torch.cuda.is_current_stream_capturing():
            return t[:M]
        _SCALE_VECS[key] = t
    return t[:M]


def concat_weights(ws) -> QuantWeight:
    """Stack linear layers that share an input along N (q|k|v, gate|up). NVFP4 parts keep
    their own fp32 global scale as a per-row scale."""
    fmt, K = ws[0].fmt, ws[0].K
    assert all(w.fmt == fmt and w.K == K for w in ws)
    data = torch.cat([w.data for w in ws], 0)
    N = sum(w.N for w in ws)
    if fmt == "bf16":
        return QuantWeight(fmt, N, K, data)
    if fmt == "fp8_block":
        assert all(w.N % 128 == 0 for w in ws[:-1]), "block-scaled parts must be 128-row aligned"
    scale = torch.cat([w.scale for w in ws], 0)
    out = QuantWeight(fmt, N, K, data, scale)
    if fmt == "nvfp4":
        out.row_gscale = torch.cat([torch.full((w.N,), w.gscale, dtype=torch.float32, device=data.device)
                                    if w.row_gscale is None else w.row_gscale * w.gscale for w in ws])
        out.gscale = 1.0
    return out


def permute_rows(w: QuantWeight, perm: torch.Tensor) -> QuantWeight:
    """Reorder output features (used to interleave gate/up rows for the SwiGLU epilogue)."""
    assert w.fmt != "fp8_block" or True
    out = QuantWeight(w.fmt, w.N, w.K, w.data[perm].contiguous(), None, w.gscale)
    if w.fmt in ("fp8_row", "nvfp4"):
        out.scale = w.scale[perm].contiguous()
    elif w.fmt == "fp8_block":
        raise ValueError("row permutation would break 128x128 scale blocks")
    if w.row_gscale is not None:
        out.row_gscale = w.row_gscale[perm].contiguous()
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows (2j, 2j+1) = (gate_j, up_j): the layout the SwiGLU GEMM epilogue pairs by lane."""
    return torch.stack([gate, up], dim=1).reshape(gate.shape[0] * 2, *gate.shape[1:])


# ----------------------------------------------------------------------------- embedding / sampling
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if not table.is_cuda:
        return table[ids.long()]
    M, hidden = ids.numel(), table.shape[1]
    out = torch.empty(M, hidden, dtype=torch.bfloat16, device=table.device)
    rt = runtime(table.device)
    _native.check(_native.lib().mb_embed(_ptr(ids), _ptr(table), _ptr(out), M, hidden, table.shape[0],
                                         _ptr(rt.status), _stream()), "embed")
    _count()
    return out


def argmax(logits: torch.Tensor, *, logprob: bool = False, mask_ids: Tuple[int, int] = (-1, -1),
           out: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None):
    """Row argmax (first maximum wins), optional top-1 log-prob and two masked ids."""
    M, V = logits.shape
    if not logits.is_cuda:
        x = logits.float().clone()
        for m in mask_ids:
            if m >= 0:
                x[:, m] = float("-inf")
        ids = x.argmax(dim=-1).to(torch.int32)
        if out is not None:
            out.copy_(ids)
        if feed is not None:
            feed.copy_(ids)
        lp = None
        if logprob:
            lp = -(torch.logsumexp(logits.float(), -1) - x.max(-1).values)
        return (ids, lp) if logprob else ids
    if out is None:
        out = torch.empty(M, dtype=torch.int32, device=logits.device)
    lp = torch.empty(M, dtype=torch.float32, device=logits.device) if logprob else None
    rc = _native.lib().mb_argmax(_ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), M, V,
                                 _ptr(out), _ptr(lp), mask_ids[0], mask_ids[1], _ptr(feed), None,
                                 _stream())
    _native.check(rc, "argmax")
    _count()
    return (out, lp) if logprob else out


def sample(logits: torch.Tensor, temperature, top_k, top_p, min_p, seed, step):
    """temperature -> top-k -> min-p -> top-p -> multinomial; rows with temperature <= 0 are
    greedy. All parameter tensors are per-row ([M]); seed/step are int64. fp32 logits."""
    M, V = logits.shape
    if not logits.is_cuda:
        return _sample_ref(logits, temperature, top_k, top_p, min_p, seed, step)
    assert logits.dtype == torch.float32
    out = torch.empty(M, dtype=torch.int32, device=logits.device)
    lp = torch.empty(M, dtype=torch.float32, device=logits.device)
    rc = _native.lib().mb_sample(_ptr(logits), logits.stride(0), M, V, _ptr(temperature), _ptr(top_k),
                                 _ptr(top_p), _ptr(min_p), _ptr(seed), _ptr(step), _ptr(out), _ptr(lp),
                                 _stream())
    _native.check(rc, "sample")
    _count()
    return out, lp


def _u01(seed: int, ctr: int) -> float:
    mask = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (ctr + 1)) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z ^= z >> 31
    return ((z >> 40) + 0.5) / 16777216.0


def sample_keep_mask(x: torch.Tensor, temp: float, k: int, p: float, mp: float) -> torch.Tensor:
    """Boolean keep-set of one fp32 logits row after top-k -> min-p -> top-p (ties kept)."""
    keep = torch.ones_like(x, dtype=torch.bool)
    V = x.numel()
    if 0 < k < V:
        kth = torch.topk(x, k).values[-1]
        keep &= x >= kth
    if mp > 0:
        keep &= x >= x.max() + temp * math.log(mp)
    if p < 1.0:
        wgt = torch.where(keep, torch.exp((x - x.max()) / temp), torch.zeros_like(x))
        need = p * wgt.sum()
        vals = torch.unique(x[keep]).flip(0)          # descending distinct values
        thr = vals[-1]
        for v in vals:
            if wgt[x >= v].sum() >= need:
                thr = v
                break
        keep &= x >= thr
    return keep


def _sample_ref(logits, temperature, top_k, top_p, min_p, seed, step):
    M, V = logits.shape
    ids = torch.empty(M, dtype=torch.int32)
    lps = torch.empty(M, dtype=torch.float32)
    for r in range(M):
        x = logits[r].float()
        t = float(temperature[r])
        lsm = torch.log_softmax(x, -1)
        if not t > 0:
            i = int(x.argmax())
        else:
            keep = sample_keep_mask(x, t, int(top_k[r]) if top_k is not None else 0,
                                    float(top_p[r]) if top_p is not None else 1.0,
                                    float(min_p[r]) if min_p is not None else 0.0)
            wgt = torch.where(keep, torch.exp((x - x.max()) / t), torch.zeros_like(x))
            cum = torch.cumsum(wgt.double(), 0)
            u = _u01(int(seed[r]), int(step[r])) * float(cum[-1])
            i = int(torch.searchsorted(cum, torch.tensor(u, dtype=torch.float64), right=True))
            i = min(i, V - 1)
        ids[r] = i
        lps[r] = lsm[i]
    return ids, lps


def apply_penalties(logits, tok, cnt, in_prompt, rep, pres, freq):
    """In-place repetition / presence / frequency penalties from per-row (token, count,
    in_prompt) triples, padded with token -1 (crates/sampling/src/penalties.rs)."""
    M, V = logits.shape
    if logits.is_cuda:
        rc = _native.lib().mb_apply_penalties(_ptr(logits), logits.stride(0), M, V, _ptr(tok), _ptr(cnt),
                                              _ptr(in_prompt), tok.shape[1], _ptr(rep), _ptr(pres),
                                              _ptr(freq), _stream())
        _native.check(rc, "penalties")
        _count()
        return logits
    for r in range(M):
        for j in range(tok.shape[1]):
            t = int(tok[r, j])
            if t < 0 or t >= V:
                continue
            c = int(cnt[r, j])
            ip = int(in_prompt[r, j]) if in_prompt is not None else 0
            v = float(logits[r, t])
            rr = float(rep[r]) if rep is not None else 1.0
            if rr != 1.0 and (c > 0 or ip):
                v = v / rr if v > 0 else v * rr
            if c > 0:
                v -= (float(pres[r]) if pres is not None else 0.0) + (float(freq[r]) if freq is not None else 0.0) * c
            logits[r, t] = v
    return logits


# ----------------------------------------------------------------------------- attention
def qk_norm_rope_kvwrite(qkv: torch.Tensor, *, Hq: int, Hkv: int, D: int, positions, slots,
                         k_cache, v_cache, q_norm_w=None, k_norm_w=None, plus_one: bool = False,
                         eps: float = 1e-6, cos=None, sin=None, q_head_stride: Optional[int] = None,
                         k_off: Optional[int] = None, v_off: Optional[int] = None,
                         k_scale=None, v_scale=None, amax=None) -> torch.Tensor:
    """Per-head q/k RMSNorm (optional) + NeoX RoPE (optional) + K/V scatter into the paged cache.
    qkv [M, *] bf16 row = q heads | k heads | v heads. Returns q [M, Hq, D] bf16. `amax`
    (fp32 [2]): running max |k| and max |v| of the rows written, for online scale calibration."""
    M = qkv.shape[0]
    qhs = q_head_stride or D
    k_off = Hq * qhs if k_off is None else k_off
    v_off = k_off + Hkv * D if v_off is None else v_off
    rot = 2 * cos.shape[1] if cos is not None else 0
    if not qkv.is_cuda:
        x = qkv.float()
        q = torch.stack([x[:, h * qhs:h * qhs + D] for h in range(Hq)], 1)
        k = x[:, k_off:k_off + Hkv * D].view(M, Hkv, D)
        v = x[:, v_off:v_off + Hkv * D].view(M, Hkv, D)
        if q_norm_w is not None:
            q = ref.bf16_round(ref.rms_norm(q, q_norm_w, eps, plus_one))
        if k_norm_w is not None:
            k = ref.bf16_round(ref.rms_norm(k, k_norm_w, eps, plus_one))
        if cos is not None:
            q = ref.apply_rope_neox(q, positions, cos, sin)
            k = ref.apply_rope_neox(k, positions, cos, sin)
        if amax is not None:
            okr = slots >= 0
            if bool(okr.any()):
                amax[0] = torch.maximum(amax[0], k[okr].abs().max())
                amax[1] = torch.maximum(amax[1], v[okr].abs().max())
        ref.kv_cache_write(k_cache, v_cache, ref.bf16_round(k) if k_cache.dtype != torch.uint8 else k,
                           v, slots, k_scale, v_scale)
        return q.to(torch.bfloat16)
    a = _native.RopeKvArgs()
    a.M, a.Hq, a.Hkv, a.D, a.rot = M, Hq, Hkv, D, rot
    a.qkv, a.qkv_ld = _ptr(qkv), qkv.stride(0)
    a.q_head_stride, a.k_off, a.v_off = qhs, k_off, v_off
    a.positions, a.slots = _ptr(positions), _ptr(slots)
    a.q_norm_w, a.k_norm_w, a.norm_plus_one, a.eps = _ptr(q_norm_w), _ptr(k_norm_w), int(plus_one), eps
    a.cos_tab, a.sin_tab = _ptr(cos), _ptr(sin)
    a.max_pos = cos.shape[0] if cos is not None else 0
    q_out = torch.empty(M, Hq, D, dtype=torch.bfloat16, device=qkv.device)
    a.q_out, a.k_cache, a.v_cache = _ptr(q_out), _ptr(k_cache), _ptr(v_cache)
    a.cache_fp8 = int(k_cache.dtype == torch.uint8)
    a.k_scale, a.v_scale = _ptr(k_scale), _ptr(v_scale)
    a.num_slots = k_cache.shape[0] * k_cache.shape[1]
    a.status = _ptr(runtime(qkv.device).status)
    a.amax = _ptr(amax)
    _native.check(_native.lib().mb_qk_norm_rope_kvwrite(C.byref(a), _stream()), "rope_kvwrite")
    _count()
    return q_out


def kv_rescale(cache: torch.Tensor, slots: torch.Tensor, old_scale: float, new_scale: torch.Tensor) -> None:
    """In place, for the listed flat slots of an e4m3 cache [blocks, block, heads, dim]: re-encode
    value * old_scale / new_scale (a per-tensor scale changed after these rows were written)."""
    nb, bs = cache.shape[0], cache.shape[1]
    row = cache.shape[2] * cache.shape[3]
    if not cache.is_cuda:
        flat = cache.view(nb * bs, row)
        ok = slots[(slots >= 0) & (slots < nb * bs)].long()
        flat[ok] = ref.to_e4m3(ref.from_e4m3(flat[ok]) * (old_scale / float(new_scale)))
        return
    _native.check(_native.lib().mb_kv_rescale(_ptr(cache), _ptr(slots), slots.numel(), row, nb * bs, float(old_scale),
                                              _ptr(new_scale), _stream()), "kv_rescale")
    _count()


_native.register_optional("mb_kv_rescale", [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_longlong, C.c_float,
                                           C.c_void_p, C.c_void_p])


# split-KV partition size (tokens); a function of nothing but this lever, so a sequence's
# partitioning -- and therefore its numerics -- never depends on the rest of the batch
_ATTN_PART_TOKENS = int(os.environ.get("METRALE_ATTN_PART_TOKENS", "0") or 0)


def configure(attn_part_tokens: Optional[int] = None) -> None:
    """Deployment constants of the kernel library. ``attn_part_tokens``: split-KV partition size;
    larger partitions amortise the per-CTA prologue and merge when the batch alone fills the GPU,
    smaller ones give short batches more CTAs. The environment lever wins over this call."""
    global _ATTN_PART_TOKENS
    if attn_part_tokens is not None and "METRALE_ATTN_PART_TOKENS" not in os.environ:
        _ATTN_PART_TOKENS = int(attn_part_tokens)


# prefill chunks of >= 128 query rows at head_dim 128 take the tcgen05 / TMEM kernel
_ATTN_TC = os.environ.get("METRALE_ATTN_TC", "1") != "0"
# 1: the V tile is staged as stored and read as an MN-major operand; 0: transposed on the way into shared memory
_ATTN_TC_VMN = int(os.environ.get("METRALE_ATTN_TC_VMN", "1"))


def paged_attention(q: torch.Tensor, k_cache, v_cache, block_table, q_start, q_len, ctx_len, *,
                    max_q_len: int, max_ctx: int, scale: float, k_scale=None, v_scale=None,
                    window: int = 0, force_mode: int = 0, part_tokens: int = 0, quant_out: float = 0.0):
    """q [T, Hq, D] bf16 -> [T, Hq, D] bf16. Caches [num_blocks, block, Hkv, D] bf16 or e4m3 bytes.
    `quant_out` > 0: return the output as an NVFP4 `Act` [T, Hq * D] quantised with that calibrated
    global scale (inside the split-KV kernel for decode-sized steps, else by a row kernel)."""
    T, Hq, D = q.shape
    if quant_out > 0.0:
        Hkv_ = k_cache.shape[2]
        fused = q.is_cuda and force_mode == 0 and (Hq // Hkv_) * max_q_len <= 16 and D % 128 == 0 and (Hq * D) % 64 == 0
        if not fused:
            o = paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, max_q_len=max_q_len,
                                max_ctx=max_ctx, scale=scale, k_scale=k_scale, v_scale=v_scale, window=window,
                                force_mode=force_mode, part_tokens=part_tokens)
            return quantize_act(o.view(T, Hq * D), "nvfp4", static_scale=quant_out)
    if not q.is_cuda:
        return ref.paged_attention(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, scale,
                                   k_scale, v_scale, window).to(torch.bfloat16)
    L = _native.lib()
    rt = runtime(q.device)
    nb, bs, Hkv, _ = k_cache.shape
    G = Hq // Hkv
    if part_tokens == 0:
        part_tokens = _ATTN_PART_TOKENS
    out = torch.empty_like(q)
    S = q_len.numel()
    if force_mode == 0 and G * max_q_len <= 32 and D == 256 and G * max_q_len > 16:
        # two row tiles do not fit the register file at head_dim 256: present every query
        # token as its own single-row sequence (causality then comes from ctx_len alone)
        return _attention_rowwise(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len,
                                  max_ctx=max_ctx, scale=scale, k_scale=k_scale, v_scale=v_scale,
                                  window=window)
    if force_mode == 3 or (force_mode == 0 and _ATTN_TC and D in (128, 256) and window == 0 and max_q_len >= 128):
        # prefill chunks: both products on tcgen05 with TMEM accumulators (csrc/attention_tc.cu)
        t = _native.AttnTcArgs()
        t.q, t.k_cache, t.v_cache, t.block_table = _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table)
        t.q_start, t.q_len, t.ctx_len = _ptr(q_start), _ptr(q_len), _ptr(ctx_len)
        t.k_scale, t.v_scale, t.out, t.status = _ptr(k_scale), _ptr(v_scale), _ptr(out), _ptr(rt.status)
        t.num_blocks, t.max_blocks, t.num_seqs, t.max_q_len = nb, block_table.stride(0), S, max_q_len
        t.Hq, t.Hkv, t.D, t.block_size, t.cache_fp8, t.scale = Hq, Hkv, D, bs, int(k_cache.dtype == torch.uint8), scale
        t.v_mn = 1 if D == 256 else _ATTN_TC_VMN
        _native.check(L.mb_attn_prefill_tc(C.byref(t), _stream()), "attn_prefill_tc")
        _count()
        return out
    a = _native.AttnArgs()
    a.q, a.k_cache, a.v_cache = _ptr(q), _ptr(k_cache), _ptr(v_cache)
    a.block_table, a.max_blocks = _ptr(block_table), block_table.stride(0)
    a.q_start, a.q_len, a.ctx_len = _ptr(q_start), _ptr(q_len), _ptr(ctx_len)
    a.num_seqs, a.max_q_len, a.max_ctx = S, max_q_len, max_ctx
    a.Hq, a.Hkv, a.D, a.block_size, a.num_blocks = Hq, Hkv, D, bs, nb
    a.scale, a.cache_fp8 = scale, int(k_cache.dtype == torch.uint8)
    a.k_scale, a.v_scale, a.out = _ptr(k_scale), _ptr(v_scale), _ptr(out)
    need = L.mb_attn_ws_bytes(T, Hq, D, max_ctx, part_tokens)
    rt.ensure_attn_ws(need)
    a.ws, a.ws_bytes, a.total_rows = _ptr(rt.attn_ws), rt.attn_ws.numel(), T
    a.part_tokens, a.window, a.force_mode, a.status = part_tokens, window, force_mode, _ptr(rt.status)
    qact = None
    if quant_out > 0.0:
        Kq = Hq * D
        qact = Act("nvfp4", T, Kq, torch.empty(T, Kq // 2, dtype=torch.uint8, device=q.device))
        qact.sf, qact.sf_k64 = _sf_buffer(q.device, T, Kq)
        qact.scale = static_scale_vec(q.device, quant_out, T)
        a.outq, a.ldq, a.outq_sf, a.outq_sf_k64, a.outq_gs = _ptr(qact.data), Kq // 2, _ptr(qact.sf), qact.sf_k64, quant_out
    _native.check(L.mb_paged_attention(C.byref(a), _stream()), "paged_attention")
    _count()
    return qact if qact is not None else out


def _attention_rowwise(q, k_cache, v_cache, block_table, q_start, q_len, ctx_len, **kw):
    T = q.shape[0]
    dev = q.device
    seq_of_row = torch.repeat_interleave(torch.arange(q_len.numel(), device=dev), q_len.long(),
                                         output_size=T)
    row_in_seq = torch.arange(T, device=dev, dtype=torch.int32) - q_start[seq_of_row]
    ctx = (ctx_len[seq_of_row] - q_len[seq_of_row] + row_in_seq + 1).to(torch.int32)
    return paged_attention(q, k_cache, v_cache, block_table[seq_of_row].contiguous(),
                           torch.arange(T, device=dev, dtype=torch.int32),
                           torch.ones(T, device=dev, dtype=torch.int32), ctx, max_q_len=1, **kw)
