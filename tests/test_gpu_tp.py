"""Tensor parallelism on 2 GPUs: the fused all-reduce + add + RMSNorm path (eager
and under CUDA graphs) against the NCCL all-reduce path and the CPU oracle."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.timeout(600)
def test_tp2_fused_allreduce_matches_nccl_and_oracle():
    import tp_worker
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.spawn(tp_worker.worker, args=(world, _free_port(), ret), nprocs=world, join=False)
    ctx.join(timeout=540)
    assert dict(ret) == {0: "ok", 1: "ok"}, "\n".join(f"[rank {k}] {v}" for k, v in ret.items())
