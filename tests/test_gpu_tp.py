"""Tensor parallelism on as many GPUs as the box has (2, 4 or 8): the fused
all-reduce + add + RMSNorm path, one-stage and two-stage, eager and under CUDA
graphs, against the NCCL all-reduce path and the CPU oracle.  On a single GPU the
same exchange is checked by tests/test_gpu_allreduce_group.py instead."""
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
def test_tp_fused_allreduce_matches_nccl_and_oracle():
    import tp_worker
    n = torch.cuda.device_count()
    world = 8 if n >= 8 else 4 if n >= 4 else 2
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.spawn(tp_worker.worker, args=(world, _free_port(), ret), nprocs=world, join=False)
    ctx.join(timeout=540)
    assert dict(ret) == {r: "ok" for r in range(world)}, \
        "\n".join(f"[rank {k}] {v}" for k, v in sorted(ret.items()))
