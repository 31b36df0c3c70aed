"""The allocation-free GEMM entry point, called through its exported C symbol.

It serves callers that may not allocate device memory (inside a stream capture, inside
another framework's memory plan, in allocator-free loops): the split-K workspace lives in a
static device array inside the library. The result must match the regular entry point (which
takes its workspace from the caller) on two calls in a row, and oversized problems must be
refused. Collected last so a failure here cannot hide any other test."""
import ctypes as C

import pytest
import torch

from metrale_inference_alpha_b200 import ops
from metrale_inference_alpha_b200.ops import _native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(act, w, out, splits):
    rt = ops.runtime(DEV)
    a = _native.GemmArgs()
    a.kind, a.M, a.N, a.K, a.ldo = ops.KIND[w.fmt], act.M, w.N, w.K, out.stride(0)
    a.W, a.X, a.out = w.data.data_ptr(), act.data.data_ptr(), out.data_ptr()
    a.alpha = 1.0
    if w.fmt == "nvfp4":
        a.sfa, a.sfb, a.sf_k64 = w.sf_tiled.data_ptr(), act.sf.data_ptr(), w.sf_k64
        a.a_scale = act.scale.data_ptr()
        a.alpha = w.gscale
    a.status = rt.status.data_ptr()
    a.force_splits, a.sm_count = splits, rt.sm_count
    return a


@pytest.mark.parametrize("fmt", ["bf16", "nvfp4"])
def test_noalloc_gemm_matches_regular_entry_point_twice(fmt):
    lib = _native.lib()
    fn = lib.mb_gemm_noalloc
    fn.argtypes = [C.POINTER(_native.GemmArgs), C.c_void_p]
    fn.restype = C.c_int
    g = torch.Generator().manual_seed(11)
    M, N, K, splits = 40, 384, 4096, 4
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        w = ops.make_weight(torch.randn(N, K, generator=g) * 0.05, fmt).to(DEV)
        act = ops.quantize_act(x, ops.ACT_FOR_WEIGHT[fmt])
        want = ops.linear(act, w, force_splits=splits, no_cluster=True)      # caller-provided workspace
        got = torch.empty_like(want)
        rc = fn(C.byref(_args(act, w, got, splits)), stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        ops.check_status(DEV)
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.float().abs().max().item()), (call, err)


def test_noalloc_gemm_refuses_oversized_workspace():
    lib = _native.lib()
    fn = lib.mb_gemm_noalloc
    fn.argtypes = [C.POINTER(_native.GemmArgs), C.c_void_p]
    fn.restype = C.c_int
    M, N, K = 128, 8192, 8192            # 64 tiles x 8 splits x 64 KiB = 32 MiB > the static array
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
    w = ops.QuantWeight("bf16", N, K, torch.zeros(N, K, dtype=torch.bfloat16, device=DEV))
    out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    act = ops.Act("bf16", M, K, x)
    rc = fn(C.byref(_args(act, w, out, 8)), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
