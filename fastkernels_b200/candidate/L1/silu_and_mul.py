"""SiLU-and-multiply.  Drop-in for SiluAndMul
(fastkernels/tasks/baseline/L1/silu_and_mul.py:13-35)."""
from __future__ import annotations

import torch.nn as nn

from fastkernels_b200 import ops


class SiluAndMul(nn.Module):
    def forward(self, x):
        shape = x.shape
        out = ops.silu_and_mul(x.reshape(-1, shape[-1]))
        return out.view(*shape[:-1], shape[-1] // 2)
