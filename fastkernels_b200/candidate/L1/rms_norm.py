"""RMSNorm / fused residual-add + RMSNorm.

Drop-in for RMSNorm (fastkernels/tasks/baseline/L1/rms_norm.py:75-164): same
constructor, parameter name (`weight`), forward(x, residual=None) returning
`out` or `(x, residual)` (both updated in place when a residual is given), and
the static forward_cuda(x, weight, eps, residual) other reference code calls.
Per-head q/k norm on a strided [N, H, D] view needs no copy.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6,
                 elementwise_affine: bool = True):
        super().__init__()
        self.hidden_size = hidden_size
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size))
        else:
            self.register_buffer("_unit_weight", torch.ones(hidden_size), persistent=False)

    @staticmethod
    def forward_cuda(x, weight, eps, residual=None):
        shape = x.shape
        compiling = torch.compiler.is_compiling()
        if compiling:
            import fastkernels_b200.torch_ops  # noqa: F401  (registers fk_b200::*)
        if residual is None:
            if x.dim() > 3 or x.dim() == 1:
                x = x.reshape(-1, shape[-1])
            y = torch.ops.fk_b200.rmsnorm(x, weight, eps) if compiling else \
                ops.rmsnorm(x, weight, eps)
            return y.view(shape)
        x2 = x.view(-1, shape[-1])
        r2 = residual.view(-1, shape[-1])
        if compiling:
            torch.ops.fk_b200.fused_add_rmsnorm(x2, r2, weight, eps)
        else:
            ops.fused_add_rmsnorm(x2, r2, weight, eps)
        return x, residual

    def forward(self, x, residual=None):
        weight = self.weight if self.elementwise_affine else self._unit_weight
        if weight.dtype != x.dtype or weight.device != x.device:
            weight = weight.to(device=x.device, dtype=x.dtype)
        return self.forward_cuda(x, weight, self.eps, residual)


share_classes(globals())
