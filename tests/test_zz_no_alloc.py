"""The allocation-free split-K GEMM entry point, called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need a GEMM: a
server whose KV cache already owns all free HBM, or a latency-critical thread that must not
call cudaMalloc (it serialises the device). For them the library keeps the split-K scratch in
a static device array. This test drives that entry point the way a C caller would - raw
pointers and a stream handle through ctypes - and checks it against the regular entry point
(caller-provided workspace) on two consecutive calls, since the calls share the scratch.

Collected last on purpose: a failure here cannot hide results of the other tests.
"""

import ctypes

import pytest
import torch

from modular_b200 import ops
from modular_b200._native import SO_PATH, lib

pytestmark = pytest.mark.gpu


def _entry():
    lib()  # make sure libtorch / the extension are loaded first
    so = ctypes.CDLL(str(SO_PATH))
    fn = so.mb_gemm_bf16_splitk_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 9 + [ctypes.c_void_p]
    err = so.mb_gemm_bf16_splitk_static_error
    err.restype = ctypes.c_int
    return fn, err


def _call(fn, x, w, y, r, splits, bn=0):
    M, K = x.shape
    N = w.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), r.data_ptr() if r is not None else None,
              M, N, K, x.stride(0), w.stride(0), y.stride(0), r.stride(0) if r is not None else 0,
              splits, bn, stream)


def test_static_scratch_gemm_matches_regular_entry_point():
    fn, err = _entry()
    torch.manual_seed(0)
    cases = [(96, 1024, 4096, 4, True), (200, 512, 2048, 3, False)]
    for M, N, K, splits, with_res in cases:  # two calls in a row on the shared scratch
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        r = torch.randn(M, N, device="cuda", dtype=torch.bfloat16) if with_res else None
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        assert _call(fn, x, w, y, r, splits) == 0
        expect = ops.linear(x, w, residual=r, splits=splits, impl="tiled")
        torch.cuda.synchronize()
        assert err() == 0
        rel = ((y.float() - expect.float()).norm() / expect.float().norm()).item()
        assert rel < 1e-2, rel
        assert torch.equal(y, expect)  # same kernels, same split: bit-identical
        # and against the plain fp32 product, so that a fault shared by both entry points cannot hide
        want = x.float() @ w.float().t() + (r.float() if r is not None else 0.0)
        assert ((y.float() - want).norm() / want.norm()).item() < 1e-2
        assert (y.float() - want).abs().max() <= 0.02 * want.abs().max() + 1e-2


def test_static_scratch_gemm_on_a_non_blocking_stream():
    """A C caller's own stream does not synchronise with the legacy stream: the error reader must still see
    the finished GEMM, and the result must match the fp32 product."""
    fn, err = _entry()
    torch.manual_seed(1)
    M, N, K, splits = 64, 2048, 8192, 4
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    y = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()      # torch creates its streams non-blocking
    rc = fn(x.data_ptr(), w.data_ptr(), y.data_ptr(), None, M, N, K, K, K, N, 0, splits, 0, s.cuda_stream)
    assert rc == 0
    assert err() == 0            # synchronises the device, the side stream included
    want = x.float() @ w.float().t()
    assert ((y.float() - want).norm() / want.norm()).item() < 1e-2


def test_static_scratch_gemm_rejects_oversize():
    fn, _ = _entry()
    x = torch.zeros(8, 64, device="cuda", dtype=torch.bfloat16)
    # 8 splits x 4096 x 4096 floats is far beyond the 4 Mi-float scratch: refused, nothing runs
    M, N = 4096, 4096
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, M, N, 64, 64, 64, N, 0, 8, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -6
