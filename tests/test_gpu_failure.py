"""Failure detection without faulting the GPU: a device-side wait whose flag
nothing ever sets must run out (bounded, 2 s), report FK_DEV_WAIT_TIMEOUT in the
status word and leave the context usable."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_that_never_signals_times_out_and_is_reported():
    from fastkernels_b200 import _lib, ops
    L = _lib.lib
    rows, cols = 4, 512
    hdr = int(L.fk_comm_header_bytes())
    total = hdr + rows * cols * 2
    bufs = []
    for _ in range(2):                      # "rank 1" is a second local buffer nobody drives
        p = C.c_void_p()
        assert L.fk_comm_alloc(total, C.byref(p)) == 0, L.fk_last_error()
        bufs.append(p.value)
    try:
        bases = (C.c_void_p * 2)(*bufs)
        residual = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
        weight = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
        out = torch.zeros_like(residual)
        status = ops.new_status("cuda")
        rc = L.fk_allreduce_add_rmsnorm(bases, 2, 0, hdr, residual.data_ptr(), cols,
                                        weight.data_ptr(), 1e-6, out.data_ptr(), cols, rows,
                                        cols, status.data_ptr(),
                                        torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.fk_last_error()
        torch.cuda.synchronize()            # returns after the 2 s bound, not never
        assert int(status.item()) & _lib.DEV_WAIT_TIMEOUT
        # the context is intact: a normal kernel still runs and is correct
        x = torch.randn(3, 256, device="cuda").to(torch.bfloat16)
        y = ops.silu_and_mul(x)
        torch.cuda.synchronize()
        assert torch.isfinite(y.float()).all()
    finally:
        for b in bufs:
            L.fk_comm_free(b)


def test_host_validation_refuses_before_launch():
    from fastkernels_b200 import _lib
    L = _lib.lib
    before = L.fk_launch_count()
    bases = (C.c_void_p * 2)(4096, 0)
    rc = L.fk_allreduce_add_rmsnorm(bases, 2, 0, int(L.fk_comm_header_bytes()), 4096, 512, 4096,
                                    1e-6, 4096, 512, 4, 512, None, None)
    assert rc == -1 and b"rank 1" in L.fk_last_error()
    rc = L.fk_allreduce_add_rmsnorm(bases, 9, 0, int(L.fk_comm_header_bytes()), 4096, 512, 4096,
                                    1e-6, 4096, 512, 4, 512, None, None)
    assert rc == -1
    assert L.fk_launch_count() == before
