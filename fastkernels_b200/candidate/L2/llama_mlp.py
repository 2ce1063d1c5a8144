"""SwiGLU MLP: gate_up_proj -> SiluAndMul -> down_proj.
Drop-in for LlamaMLP (fastkernels/tasks/baseline/L2/llama_mlp.py:16-38)."""
from __future__ import annotations

import torch.nn as nn

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

    def forward(self, x):
        return self.down_proj(self.act_fn(self.gate_up_proj(x)))


share_classes(globals())
