"""fk_gemm_bf16_static: the projection for hosts that may not allocate device
memory (plugins inside someone else's memory pool, code that runs while a stream
is being captured).  Its scratch is an array inside the library, so the call
takes no workspace.  Checked here through the C-ABI: two calls in a row must give
exactly what fk_gemm_bf16 gives with a caller-provided workspace (same kernel,
fixed summation order, hence bit-identical), and a batch beyond the built-in
limit must be refused with a clear message rather than run.

This file sorts last on purpose: a run that stops at the first failure has
already executed every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(L, x, w, bias, y):
    return L.fk_gemm_bf16_static(
        x.data_ptr(), x.stride(0), w.data_ptr(), None if bias is None else bias.data_ptr(),
        y.data_ptr(), y.stride(0), x.shape[0], w.shape[0], x.shape[1], None,
        torch.cuda.current_stream().cuda_stream)


def test_static_scratch_gemm_matches_workspace_gemm_twice():
    from fastkernels_b200 import _lib, ops
    L = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(11)
    for (m, n, k, with_bias) in [(64, 4096, 4096, False), (7, 1000, 512, True)]:
        x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        b = torch.randn(n, generator=g, device="cuda").to(torch.bfloat16) if with_bias else None
        want = ops.gemm_bf16(x, w, b)                      # existing entry point
        for _ in range(2):                                 # two calls in a row
            got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            rc = _call_static(L, x, w, b, got)
            assert rc == 0, L.fk_last_error()
            torch.cuda.synchronize()
            assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        # and the shared scratch is left clean for the next caller
        again = ops.gemm_bf16(x, w, b)
        assert torch.equal(again.view(torch.int16), want.view(torch.int16))


def test_static_scratch_gemm_rejects_oversized_batch():
    from fastkernels_b200 import _lib
    L = _lib.lib
    x = torch.zeros((65, 64), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    y = torch.zeros((65, 128), dtype=torch.bfloat16, device="cuda")
    before = L.fk_launch_count()
    rc = _call_static(L, x, w, None, y)
    assert rc == -2
    msg = L.fk_last_error().decode()
    assert "m <= 64" in msg and "fk_gemm_bf16" in msg
    assert L.fk_launch_count() == before                   # nothing was launched
