"""SiLU-and-multiply.  Drop-in for SiluAndMul
(fastkernels/tasks/baseline/L1/silu_and_mul.py:13-35)."""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class SiluAndMul(nn.Module):
    def forward(self, x):
        shape = x.shape
        if torch.compiler.is_compiling():
            import fastkernels_b200.torch_ops  # noqa: F401  (registers fk_b200::*)
            out = torch.ops.fk_b200.silu_and_mul(x.reshape(-1, shape[-1]))
        else:
            out = ops.silu_and_mul(x.reshape(-1, shape[-1]))
        return out.view(*shape[:-1], shape[-1] // 2)


share_classes(globals())
