"""Dense projection on the tcgen05 decode GEMM.

Drop-in for Matmul / Linear (fastkernels/tasks/baseline/L1/linear.py:13-37):
Matmul.forward(input, weight, bias=None) = input @ weight.T (+ bias).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class Matmul(nn.Module):
    def forward(self, input, weight, bias=None):
        shape = input.shape
        x = input.reshape(-1, shape[-1])
        if torch.compiler.is_compiling():
            import fastkernels_b200.torch_ops  # noqa: F401  (registers fk_b200::*)
            y = torch.ops.fk_b200.gemm_bf16(x, weight, bias)
        else:
            y = ops.gemm_bf16(x, weight, bias)
        return y.view(*shape[:-1], weight.shape[0])


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        self.matmul = Matmul()

    def forward(self, input):
        return self.matmul(input, self.weight, self.bias)


share_classes(globals())
