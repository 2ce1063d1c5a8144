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
