"""Fused all-reduce + residual add + RMSNorm for 2, 4 and 8 ranks on ONE GPU.

Every rank's communication buffer lives on the same device and all ranks run in
one cooperative launch (fk_allreduce_add_rmsnorm_group): the same row routine,
flags, epochs and slot alternation as the per-rank kernel of a real
tensor-parallel group, with the peer loads and stores landing in local memory.
Kernels that wait for each other are never issued as separate launches on one
GPU.  Checked against the oracle's restatement of the reference's sum
(allreduce.cu:184-191) + fused add RMSNorm: new residual bit-exact, output within
one bf16 step, all ranks bit-identical, one-stage and two-stage identical.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from gpu_util import assert_bf16_close, dev, host_bits, host_f32
from oracle import decode_oracle as O

pytestmark = pytest.mark.gpu


class Group:
    """nranks communication buffers on the current device."""

    def __init__(self, nranks, max_rows, cols):
        from fastkernels_b200 import _lib
        self.L = _lib.lib
        self.n, self.cols = nranks, cols
        self.hdr = int(self.L.fk_comm_header_bytes())
        self.slot_bytes = (max_rows * cols * 2 + 255) // 256 * 256
        self.total = self.hdr + 4 * self.slot_bytes      # 2 slots + 2 staging areas
        self.bufs = []
        for _ in range(nranks):
            p = C.c_void_p()
            assert self.L.fk_comm_alloc(self.total, C.byref(p)) == 0, self.L.fk_last_error()
            self.bufs.append(p.value)
        self.bases = (C.c_void_p * nranks)(*self.bufs)

    def close(self):
        for b in self.bufs:
            self.L.fk_comm_free(b)

    def slot(self, rank, slot, rows):
        class Mem:
            pass
        m = Mem()
        m.__cuda_array_interface__ = {
            "shape": (rows * self.cols,), "typestr": "<i2",
            "data": (self.bufs[rank] + self.hdr + slot * self.slot_bytes, False), "version": 2}
        return torch.as_tensor(m, device="cuda").view(torch.bfloat16).view(rows, self.cols)

    def run(self, slot, rows, residuals, weight, eps, outs, status, two_stage):
        res = (C.c_void_p * self.n)(*[t.data_ptr() for t in residuals])
        out = (C.c_void_p * self.n)(*[t.data_ptr() for t in outs])
        staging = self.hdr + (2 + slot) * self.slot_bytes if two_stage else 0
        rc = self.L.fk_allreduce_add_rmsnorm_group(
            self.bases, self.n, self.hdr + slot * self.slot_bytes, staging, res, self.cols,
            weight.data_ptr(), eps, out, self.cols, rows, self.cols, status.data_ptr(),
            torch.cuda.current_stream().cuda_stream)
        assert rc == 0, self.L.fk_last_error()


@pytest.mark.parametrize("nranks", [2, 4, 8])
# 128 rows x 8 ranks is more blocks than the device holds at once: blocks then walk
# several rows each
@pytest.mark.parametrize("rows,cols", [(1, 4096), (64, 4096), (128, 8192), (37, 512)])
def test_group_allreduce_matches_oracle(nranks, rows, cols):
    from fastkernels_b200 import ops
    rs = np.random.RandomState(1000 * nranks + rows + cols)
    grp = Group(nranks, rows, cols)
    try:
        status = ops.new_status("cuda")
        w = cases.randn_bf16(rs, (cols,), 0.02) + 1.0
        w = O.bf16_round(w)
        wd = dev(w)
        residual = cases.randn_bf16(rs, (rows, cols))
        # each algorithm keeps its own running residual; they must stay bit-equal
        res_dev = {alg: [dev(residual) for _ in range(nranks)] for alg in (False, True)}
        res_ref = residual
        # three consecutive calls alternating slots, both algorithms after one another
        # on the same buffers (mixed sequences are allowed)
        for call in range(3):
            slot = call & 1
            parts = [cases.randn_bf16(rs, (rows, cols), 0.5) for _ in range(nranks)]
            want_out, want_res = O.allreduce_add_rmsnorm(parts, res_ref, w, 1e-6)
            got = {}
            for two_stage in (False, True):
                for r in range(nranks):
                    grp.slot(r, slot, rows).copy_(dev(parts[r]))
                outs = [torch.full((rows, cols), float("nan"), dtype=torch.bfloat16,
                                   device="cuda") for _ in range(nranks)]
                grp.run(slot, rows, res_dev[two_stage], wd, 1e-6, outs, status, two_stage)
                torch.cuda.synchronize()
                assert int(status.item()) == 0, f"device status {int(status.item())}"
                got[two_stage] = outs
                for r in range(nranks):
                    # residual: bit-exact against the oracle; out: one bf16 step
                    assert np.array_equal(host_bits(res_dev[two_stage][r]),
                                          O.bf16_round_bits(want_res)), (call, two_stage, r)
                    assert_bf16_close(outs[r], want_out, max_ulp=1, frac=0.03)
                    assert torch.equal(outs[r].view(torch.int16), outs[0].view(torch.int16)), \
                        f"rank {r} differs from rank 0 (call {call}, two_stage={two_stage})"
            assert torch.equal(got[False][0].view(torch.int16), got[True][0].view(torch.int16))
            res_ref = want_res
    finally:
        grp.close()


def test_two_stage_rule():
    """One stage at every decode payload (measured faster on B200); two stages on 8
    ranks from 4 MiB on (prefill chunks)."""
    from fastkernels_b200 import _lib
    f = _lib.lib.fk_allreduce_two_stage_preferred
    assert f(2, 512, 8192) == 0 and f(4, 512, 8192) == 0
    assert f(8, 128, 8192) == 0                       # the 70B-shape decode payload, 2 MiB
    assert f(8, 256, 8192) == 1 and f(8, 255, 8192) == 0


@pytest.mark.parametrize("nranks", [2, 4, 8])
# k sizes that take the cluster split-K (push and pull reductions) and the stream-K
# schedule of the projection: all three epilogues store into the receive areas
@pytest.mark.parametrize("rows,cols,k", [(64, 4096, 1024), (128, 4096, 512), (5, 512, 192),
                                         (64, 12288, 256), (1, 4096, 4096)])
def test_pushed_exchange_matches_pulled_and_oracle(nranks, rows, cols, k):
    """The row-parallel projection of every rank stores its tiles straight into all
    ranks' receive areas (fk_gemm_bf16_push); fk_allreduce_add_rmsnorm_pushed then
    reads only its own buffer.  On one GPU the "ranks" run one after the other
    (nothing waits on a later launch: every word a norm kernel polls for was written
    by an earlier one).  Same bits as the projection into a slot + the oracle's
    all-reduce + add + RMSNorm, for three calls on alternating slots."""
    from fastkernels_b200 import _lib, ops
    L = _lib.lib
    rs = np.random.RandomState(7 * nranks + rows + cols + k)
    hdr = int(L.fk_comm_header_bytes())
    area = (rows * cols * 4 + 255) // 256 * 256
    total = hdr + 2 * nranks * area
    bufs = []
    try:
        for _ in range(nranks):
            p = C.c_void_p()
            assert L.fk_comm_alloc(total, C.byref(p)) == 0, L.fk_last_error()
            bufs.append(p.value)
        status = ops.new_status("cuda")
        w_norm = O.bf16_round(cases.randn_bf16(rs, (cols,), 0.02) + 1.0)
        wd = dev(w_norm)
        residual = cases.randn_bf16(rs, (rows, cols))
        res_dev = [dev(residual) for _ in range(nranks)]
        res_ref = residual
        epoch_off = int(L.fk_comm_epoch_offset())
        for call in range(3):
            slot = call & 1
            xs = [dev(cases.randn_bf16(rs, (rows, k), 0.5)) for _ in range(nranks)]
            ws = [dev(cases.randn_bf16(rs, (cols, k), 0.05)) for _ in range(nranks)]
            bias = dev(cases.randn_bf16(rs, (cols,), 0.1))
            # what each rank's projection writes into a slot on the pulled path
            parts = [host_f32(ops.gemm_bf16(xs[r], ws[r], bias if r == 0 else None))
                     for r in range(nranks)]
            want_out, want_res = O.allreduce_add_rmsnorm(parts, res_ref, w_norm, 1e-6)
            for r in range(nranks):           # sender r -> its area in every buffer
                dst = (C.c_void_p * nranks)(*[b + hdr + (slot * nranks + r) * area for b in bufs])
                ops.gemm_bf16_push(xs[r], ws[r], bias if r == 0 else None, dst, nranks,
                                   bufs[r] + epoch_off, status=status)
            outs = [torch.full((rows, cols), float("nan"), dtype=torch.bfloat16, device="cuda")
                    for _ in range(nranks)]
            for r in range(nranks):
                rc = L.fk_allreduce_add_rmsnorm_pushed(
                    bufs[r], nranks, hdr + slot * nranks * area, area, res_dev[r].data_ptr(), cols,
                    wd.data_ptr(), 1e-6, outs[r].data_ptr(), cols, rows, cols, status.data_ptr(),
                    torch.cuda.current_stream().cuda_stream)
                assert rc == 0, L.fk_last_error()
            torch.cuda.synchronize()
            assert int(status.item()) == 0, f"device status {int(status.item())}"
            for r in range(nranks):
                assert np.array_equal(host_bits(res_dev[r]), O.bf16_round_bits(want_res)), (call, r)
                assert_bf16_close(outs[r], want_out, max_ulp=1, frac=0.03)
                assert torch.equal(outs[r].view(torch.int16), outs[0].view(torch.int16))
            res_ref = want_res
    finally:
        for b in bufs:
            L.fk_comm_free(b)


def test_pushed_exchange_wait_is_bounded():
    """Nothing was pushed: the norm kernel gives up after its 2 s budget, reports
    FK_DEV_WAIT_TIMEOUT and returns; the context stays usable."""
    from fastkernels_b200 import _lib, ops
    L = _lib.lib
    hdr = int(L.fk_comm_header_bytes())
    rows, cols, area = 2, 256, 4096
    p = C.c_void_p()
    assert L.fk_comm_alloc(hdr + 2 * area, C.byref(p)) == 0
    try:
        status = ops.new_status("cuda")
        res = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
        out = torch.empty_like(res)
        w = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
        rc = L.fk_allreduce_add_rmsnorm_pushed(p.value, 2, hdr, area, res.data_ptr(), cols,
                                               w.data_ptr(), 1e-6, out.data_ptr(), cols, rows,
                                               cols, status.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
        assert rc == 0, L.fk_last_error()
        torch.cuda.synchronize()
        assert int(status.item()) & 4
        assert torch.equal(ops.rmsnorm(res + 1, w, 1e-6), ops.rmsnorm(res + 1, w, 1e-6))
    finally:
        L.fk_comm_free(p.value)


def test_push_rule():
    from fastkernels_b200 import _lib
    f = _lib.lib.fk_allreduce_push_preferred
    assert f(2, 64, 4096) == 1 and f(4, 64, 4096) == 1        # 1 and 3 MiB on the wire
    assert f(8, 64, 4096) == 0 and f(4, 128, 8192) == 0       # 7 and 12 MiB: pulled
    assert f(1, 64, 4096) == 0
