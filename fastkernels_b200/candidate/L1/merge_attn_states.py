"""Log-sum-exp merge of two partial attention results.

Drop-in for merge_attn_states / MergeAttnStates
(fastkernels/tasks/baseline/L1/merge_attn_states.py:32-122): same function
signature (output and output_lse written in place), same module.  fp8 output
(`output_scale`) is not on this path.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


def merge_attn_states(output, prefix_output, prefix_lse, suffix_output, suffix_lse,
                      output_lse=None, prefill_tokens_with_context=None,
                      output_scale=None) -> None:
    if output_scale is not None:
        raise NotImplementedError("fp8 output is not on this path")
    ops.merge_attn_states(output, prefix_output, prefix_lse, suffix_output, suffix_lse,
                          output_lse, prefill_tokens_with_context)


class MergeAttnStates(nn.Module):
    """Online softmax merge of two attention partitions."""

    def forward(self, output, prefix_output, prefix_lse, suffix_output, suffix_lse,
                output_lse=None) -> None:
        merge_attn_states(output, prefix_output, prefix_lse, suffix_output, suffix_lse,
                          output_lse)


share_classes(globals())
