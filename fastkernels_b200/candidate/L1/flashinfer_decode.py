"""Paged GQA decode attention over an HND page table.

Drop-in for TRTLLMDecode (fastkernels/tasks/baseline/L1/flashinfer_decode.py:44-107),
the decode op the reference selects by default on Blackwell (HND layout, page size
16; fastkernels/infra/context.py:57-67): same constructor, same
forward(q, k_cache, v_cache, cache_seqlens, block_table=..., softmax_scale=...,
causal=..., max_seq_len=..., s_aux=..., window_size=...) -> [N, Hq, D], and the
`_workspace` / `prime_sinks` surface the attention layer touches
(fastkernels/tasks/baseline/L2/attention_impl.py:289-311).  It runs the same
split-KV kernel as FlashAttnDecode with the HND tensor map; unlike the reference
call it needs neither contiguous q nor contiguous block tables.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class TRTLLMDecode(nn.Module):
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
        self._max_splits = 32
        self._fk_workspace: torch.Tensor | None = None
        self._ws_batch = 0
        self._status: torch.Tensor | None = None

    def prime_sinks(self, sinks) -> None:
        if sinks is not None:
            raise NotImplementedError("attention sinks are not on this path")

    def preallocate(self, max_batch_size: int, device) -> None:
        if self._fk_workspace is None or self._ws_batch < max_batch_size:
            n = ops.attn_workspace_bytes(max_batch_size, self.num_qo_heads, self.head_dim,
                                         self._max_splits)
            self._fk_workspace = torch.empty(n, dtype=torch.uint8, device=device)
            self._ws_batch = max_batch_size
        if self._status is None:
            self._status = ops.new_status(device)

    def forward(self, q, k_cache, v_cache, cache_seqlens=None, block_table=None,
                softmax_scale=None, causal=True, max_seq_len=None, s_aux=None,
                window_size=None, **kwargs):
        if s_aux is not None or (window_size is not None and tuple(window_size) != (-1, -1)):
            raise NotImplementedError("attention sinks / sliding windows are not on this path")
        planned = bool(kwargs.pop("plan_ready", False))
        self.preallocate(q.shape[0], q.device)
        return ops.paged_decode_attn(
            q, k_cache, v_cache, cache_seqlens, block_table,
            softmax_scale if softmax_scale is not None else self.sm_scale,
            self._fk_workspace, self._max_splits, status=self._status, planned=planned,
            kv_layout="HND")


share_classes(globals())
