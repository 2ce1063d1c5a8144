"""Tensor-parallel sum.  Drop-in for AllReduce
(fastkernels/tasks/baseline/L1/allreduce.py:37-55) on its NCCL path
(dist.all_reduce, graph-capturable; allreduce.py:47,54): in place, returns the
same tensor.  NCCL runs the reduction over NVLink 5 / NVSwitch."""
from __future__ import annotations

import torch.distributed as dist
import torch.nn as nn
from fastkernels_b200.candidate import share_classes


class AllReduce(nn.Module):
    def forward(self, tensor):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(tensor)
        return tensor


share_classes(globals())
