"""ctypes binding of ``libmetrale_b200.so`` (the in-tree sm_100a kernel library).

The structures below mirror the ``extern "C"`` argument structs in ``csrc/*.cu`` field for
field. ``lib()`` raises if the shared object is missing: on a machine with a GPU the CUDA
path is the only path, there is no silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libmetrale_b200.so"
_lib = None

c_void_p, c_int, c_float, c_ll, c_size_t = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_size_t


class GemmArgs(C.Structure):
    _fields_ = [
        ("kind", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("ldo", c_int), ("a_ld", c_int),
        ("W", c_void_p), ("X", c_void_p), ("out", c_void_p), ("residual", c_void_p),
        ("w_scale", c_void_p), ("a_scale", c_void_p), ("alpha", c_float),
        ("sfa", c_void_p), ("sfb", c_void_p), ("sf_k64", c_int),
        ("epilogue", c_int), ("out_f32", c_int),
        ("ws", c_void_p), ("ws_bytes", c_size_t), ("status", c_void_p),
        ("force_tn", c_int), ("force_splits", c_int), ("sm_count", c_int), ("flags", c_int), ("timing_trace", c_void_p), ("no_cluster", c_int),
        ("outq", c_void_p), ("ldq", c_int), ("outq_sf", c_void_p), ("outq_sf_k64", c_int), ("outq_gs", c_float),
        ("tile_expert", c_void_p), ("tile_row0", c_void_p), ("tile_nrows", c_void_p),
        ("n_per_expert", c_int), ("max_tiles", c_int),
    ]


class RowArgs(C.Structure):
    _fields_ = [
        ("M", c_int), ("K", c_int), ("in_mode", c_int), ("out_mode", c_int),
        ("x", c_void_p), ("x_ld", c_ll), ("residual", c_void_p), ("residual_out", c_void_p),
        ("w", c_void_p), ("w_plus_one", c_int), ("eps", c_float),
        ("gate", c_void_p), ("gate_ld", c_ll),
        ("head_dim", c_int), ("gate_head_stride", c_int), ("gate_head_off", c_int), ("group", c_int),
        ("xf32", c_void_p), ("out", c_void_p), ("out_ld", c_ll),
        ("out_bf16", c_void_p), ("out_bf16_ld", c_ll),
        ("scale", c_void_p), ("scale_ld", c_int), ("sf", c_void_p), ("sf_k64", c_int), ("static_gs", c_float),
        ("row_index", c_void_p),
    ]


class AttnTcArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("block_table", c_void_p),
        ("q_start", c_void_p), ("q_len", c_void_p), ("ctx_len", c_void_p), ("k_scale", c_void_p), ("v_scale", c_void_p),
        ("out", c_void_p), ("status", c_void_p), ("num_blocks", c_ll),
        ("max_blocks", c_int), ("num_seqs", c_int), ("max_q_len", c_int), ("Hq", c_int), ("Hkv", c_int), ("D", c_int),
        ("block_size", c_int), ("cache_fp8", c_int), ("scale", c_float), ("v_mn", c_int),
    ]


class A16Args(C.Structure):
    _fields_ = [
        ("kind", c_int), ("M", c_int), ("N", c_int), ("K", c_int), ("ldx", c_int), ("ldo", c_int),
        ("swiglu", c_int), ("scale_ld", c_int),
        ("W", c_void_p), ("scale", c_void_p), ("row_gscale", c_void_p), ("x", c_void_p),
        ("residual", c_void_p), ("out", c_void_p), ("out_f32", c_void_p),
        ("gscale", c_float), ("n_lo", c_int), ("rows", c_int),
    ]


class RopeKvArgs(C.Structure):
    _fields_ = [
        ("M", c_int), ("Hq", c_int), ("Hkv", c_int), ("D", c_int), ("rot", c_int),
        ("qkv", c_void_p), ("qkv_ld", c_ll),
        ("q_head_stride", c_int), ("k_off", c_int), ("v_off", c_int),
        ("positions", c_void_p), ("slots", c_void_p),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("norm_plus_one", c_int), ("eps", c_float),
        ("cos_tab", c_void_p), ("sin_tab", c_void_p), ("max_pos", c_int),
        ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p), ("cache_fp8", c_int),
        ("k_scale", c_void_p), ("v_scale", c_void_p), ("num_slots", c_ll), ("status", c_void_p),
        ("amax", c_void_p),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("block_table", c_void_p), ("max_blocks", c_int),
        ("q_start", c_void_p), ("q_len", c_void_p), ("ctx_len", c_void_p),
        ("num_seqs", c_int), ("max_q_len", c_int), ("max_ctx", c_int),
        ("Hq", c_int), ("Hkv", c_int), ("D", c_int), ("block_size", c_int),
        ("num_blocks", c_ll), ("scale", c_float), ("cache_fp8", c_int),
        ("k_scale", c_void_p), ("v_scale", c_void_p), ("out", c_void_p),
        ("ws", c_void_p), ("ws_bytes", c_size_t), ("total_rows", c_int),
        ("part_tokens", c_int), ("window", c_int), ("force_mode", c_int), ("status", c_void_p),
        ("outq", c_void_p), ("ldq", c_int), ("outq_sf", c_void_p), ("outq_sf_k64", c_int), ("outq_gs", c_float),
    ]


def available() -> bool:
    return LIB_PATH.exists()


def check_arch(capability=None) -> None:
    """The library holds sm_100a code only (tcgen05 / TMEM have no forward-compatible PTX): refuse
    any other device up front instead of failing in the first launch with "no kernel image"."""
    if capability is None:
        import torch
        if not torch.cuda.is_available():
            return
        capability = torch.cuda.get_device_capability()
    if tuple(capability) != (10, 0):
        raise RuntimeError(f"this build targets NVIDIA B200 (sm_100a); the current device reports sm_{capability[0]}{capability[1]}. "
                           "Architecture-specific sm_100a code does not run on other architectures.")


def lib():
    """Load (once) and return the kernel library; raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        if os.environ.get("METRALE_B200_AUTOBUILD", "1") == "1":
            from . import build as _build
            _build.build()
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m metrale_inference_alpha_b200.ops.build`")
    check_arch()
    L = C.CDLL(str(LIB_PATH))
    P = C.POINTER
    L.mb_gemm.argtypes = [P(GemmArgs), c_void_p]
    L.mb_gemm.restype = c_int
    for fn in (L.mb_a16_gemv, L.mb_a16_dequant):
        fn.argtypes = [P(A16Args), c_void_p]
        fn.restype = c_int
    L.mb_attn_prefill_tc.argtypes = [P(AttnTcArgs), c_void_p]
    L.mb_attn_prefill_tc.restype = c_int
    L.mb_gguf_dequant.argtypes = [c_int, c_void_p, c_ll, c_void_p, c_void_p]
    L.mb_gguf_dequant.restype = c_int
    L.mb_gemm_counter_bytes.argtypes = []
    L.mb_gemm_counter_bytes.restype = c_size_t
    L.mb_row_op.argtypes = [P(RowArgs), c_void_p]
    L.mb_row_op.restype = c_int
    L.mb_sf_repack.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    L.mb_sf_repack.restype = c_int
    L.mb_add_inplace.argtypes = [c_void_p, c_void_p, c_ll, c_void_p]
    L.mb_add_inplace.restype = c_int
    L.mb_embed.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]
    L.mb_embed.restype = c_int
    L.mb_qk_norm_rope_kvwrite.argtypes = [P(RopeKvArgs), c_void_p]
    L.mb_qk_norm_rope_kvwrite.restype = c_int
    L.mb_paged_attention.argtypes = [P(AttnArgs), c_void_p]
    L.mb_paged_attention.restype = c_int
    L.mb_attn_ws_bytes.argtypes = [c_int, c_int, c_int, c_int, c_int]
    L.mb_attn_ws_bytes.restype = c_size_t
    L.mb_argmax.argtypes = [c_void_p, c_int, c_ll, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                            c_void_p, c_void_p, c_void_p]
    L.mb_argmax.restype = c_int
    L.mb_sample.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    L.mb_sample.restype = c_int
    L.mb_apply_penalties.argtypes = [c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    L.mb_apply_penalties.restype = c_int
    for name, argtypes in _OPTIONAL.items():
        fn = getattr(L, name, None)
        if fn is not None:
            fn.argtypes = argtypes
            fn.restype = c_int
    _lib = L
    return L


# entry points added by later kernel files; bound when present
_OPTIONAL: dict = {}


def register_optional(name: str, argtypes) -> None:
    _OPTIONAL[name] = argtypes
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int


class KernelError(RuntimeError):
    pass


_CODES = {-1: "bad argument", -2: "unsupported shape/format", -3: "workspace too small or size beyond limit",
          -4: "CUDA driver entry point unavailable"}


# Launch trace: while a recorder list is installed, every launcher call appends its name, so two
# runs (or a graph capture and an eager step) can be compared launch by launch. Role of the
# reference's launch trace diff and kernel-resolution audit (crates/telemetry/src/launch_trace.rs).
_trace = None


class launch_trace:
    """``with launch_trace() as names: ...`` collects the name of every kernel launcher called."""

    def __enter__(self):
        global _trace
        self._prev, self.names = _trace, []
        _trace = self.names
        return self.names

    def __exit__(self, *exc):
        global _trace
        _trace = self._prev
        return False


def diff_traces(a, b):
    """First position at which two launch traces differ, as (index, name_a, name_b), or None."""
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            return i, x, y
    if len(a) != len(b):
        i = min(len(a), len(b))
        return i, a[i] if i < len(a) else None, b[i] if i < len(b) else None
    return None


_launch_hook = None
_audit = None          # dict name -> launches while a kernel audit is on (utils/kernel_audit.py)


def set_launch_hook(fn) -> None:
    """fn(kernel launcher name) is called after every launch (telemetry level "kernel")."""
    global _launch_hook
    _launch_hook = fn


def check(rc: int, what: str) -> None:
    if _audit is not None and rc == 0:
        name = what.split("[", 1)[0]
        _audit[name] = _audit.get(name, 0) + 1
    if _trace is not None:
        _trace.append(what.split("[", 1)[0])
    if _launch_hook is not None and rc == 0:
        _launch_hook(what.split("[", 1)[0])
    if rc != 0:
        msg = _CODES.get(rc, f"CUDA error {rc}")
        raise KernelError(f"{what}: {msg}")
