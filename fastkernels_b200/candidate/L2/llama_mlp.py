"""SwiGLU MLP: gate_up_proj -> SiluAndMul -> down_proj.
Drop-in for LlamaMLP (fastkernels/tasks/baseline/L2/llama_mlp.py:16-38)."""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate.L1.silu_and_mul import SiluAndMul
from fastkernels_b200.candidate.L2.parallel_linear import (MergedColumnParallelLinear,
                                                            RowParallelLinear)
from fastkernels_b200.candidate import share_classes


class LlamaMLP(nn.Module):
    def __init__(self, config, quant_config: dict | None = None,
                 hidden_size: int | None = None, intermediate_size: int | None = None,
                 reduce_results: bool = True):
        super().__init__()
        h = hidden_size if hidden_size is not None else config.hidden_size
        i = intermediate_size if intermediate_size is not None else config.intermediate_size
        self.gate_up_proj = MergedColumnParallelLinear(h, [i] * 2, quant_config=quant_config)
        self.down_proj = RowParallelLinear(i, h, quant_config=quant_config,
                                           reduce_results=reduce_results)
        self.down_proj.comm_slot = 1
        self.act_fn = SiluAndMul()
        # build-only switch (not a reference argument): run gate_up + SiLU as one kernel
        self.fused_act = True

    def forward(self, x):
        gu = self.gate_up_proj
        if (self.fused_act and x.dim() == 2 and x.is_cuda and x.dtype == torch.bfloat16
                and not torch.compiler.is_compiling()
                and ops.gemm_silu_mul_fusable(x.shape[0], gu.weight.shape[0], x.shape[1])):
            # gate/up projection and SiLU-and-multiply in one launch (same rounding
            # points as the two ops)
            return self.down_proj(ops.gemm_silu_mul(x, gu.weight, gu.bias))
        return self.down_proj(self.act_fn(gu(x)))


share_classes(globals())
