"""Variable-length prefill attention over the HND paged pool.

Drop-in for TRTLLMPrefill (fastkernels/tasks/baseline/L1/flashinfer_prefill.py:
15-100), the prefill op the reference pairs with TRTLLMDecode on Blackwell: same
constructor, same cu_seqlens-based forward as FlashAttnPrefill, `_workspace` /
`prime_sinks` surface (fastkernels/tasks/baseline/L2/attention_impl.py:289-311).
Runs the same tcgen05 kernel as FlashAttnPrefill with the HND tensor map; needs
neither contiguous q nor contiguous block tables, and no scratch buffer.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class TRTLLMPrefill(nn.Module):
    def __init__(self, num_qo_heads: int, num_kv_heads: int, head_dim: int,
                 workspace: torch.Tensor | None = None):
        super().__init__()
        self.num_qo_heads = num_qo_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.sm_scale = head_dim ** -0.5
        self._workspace = workspace      # the reference's 512 MiB scratch: not needed
        self._sinks_fp32 = None
        self._sinks_src = None
        self._status: torch.Tensor | None = None

    def prime_sinks(self, sinks) -> None:
        if sinks is not None:
            raise NotImplementedError("attention sinks are not on this path")

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                softmax_scale=None, causal=True, block_table=None, s_aux=None,
                window_size=None, **kwargs):
        if s_aux is not None or (window_size is not None and tuple(window_size) != (-1, -1)):
            raise NotImplementedError("attention sinks / sliding windows are not on this path")
        if self._status is None:
            self._status = ops.new_status(q.device)
        tq = q.shape[0]
        q3 = q.view(tq, self.num_qo_heads, self.head_dim)
        if block_table is None:
            k = k.view(k.shape[0], self.num_kv_heads, self.head_dim)
            v = v.view(v.shape[0], self.num_kv_heads, self.head_dim)
        elif block_table.dtype != torch.int32:
            block_table = block_table.to(torch.int32)
        to32 = lambda t: t if t.dtype == torch.int32 else t.to(torch.int32)  # noqa: E731
        return ops.prefill_attn(
            q3, k, v, to32(cu_seqlens_q), to32(cu_seqlens_k), int(max_seqlen_q),
            softmax_scale if softmax_scale is not None else self.sm_scale, causal=causal,
            block_table=block_table, kv_layout="HND", status=self._status)


share_classes(globals())
