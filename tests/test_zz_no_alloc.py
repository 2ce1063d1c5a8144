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


# (m, n, k, bias).  The first two shapes have few weight tiles, so the planner
# splits k inside thread-block clusters and the scratch array is not touched; the
# last three have more tiles than half the SMs, which selects the stream-K
# schedule: partial tiles and flags go through the built-in array.
SHAPES = [(64, 4096, 4096, False), (7, 1000, 512, True),
          (64, 24576, 4096, False), (5, 12800, 4096, True), (33, 24576, 1024, True)]


def test_static_scratch_gemm_matches_workspace_gemm_twice():
    from fastkernels_b200 import _lib, ops
    L = _lib.lib
    g = torch.Generator(device="cuda").manual_seed(11)
    for (m, n, k, with_bias) in SHAPES:
        w = (torch.randn((n, k), generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        b = torch.randn(n, generator=g, device="cuda").to(torch.bfloat16) if with_bias else None
        # two calls in a row on DIFFERENT activations: a flag left raised or a
        # partial tile picked up from the previous call would change the second
        xs = [torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
              for _ in range(2)]
        wants = [ops.gemm_bf16(x, w, b) for x in xs]       # existing entry point
        gots = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
                for _ in range(2)]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for x, got in zip(xs, gots):
            rc = _call_static(L, x, w, b, got)
            assert rc == 0, L.fk_last_error()
        torch.cuda.synchronize()
        # the entry point allocates nothing: device memory in use is unchanged (the
        # outputs were made before the first reading; a stream-K workspace for
        # this batch would be 5 MiB, the allowance is for driver bookkeeping)
        assert free_before - torch.cuda.mem_get_info()[0] < (1 << 20)
        for got, want in zip(gots, wants):
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, n, k)
        # and a third call, on the first activations again, still agrees
        got = torch.empty_like(gots[0])
        assert _call_static(L, xs[0], w, b, got) == 0, L.fk_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), wants[0].view(torch.int16))


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
