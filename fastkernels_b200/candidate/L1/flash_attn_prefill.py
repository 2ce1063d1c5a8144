"""Variable-length prefill attention (dense K/V or the paged NHD pool).

Drop-in for FlashAttnPrefill (fastkernels/tasks/baseline/L1/flash_attn_prefill.py:
18-74): same constructor, same forward(q, k, v, cu_seqlens_q, cu_seqlens_k,
max_seqlen_q, max_seqlen_k, softmax_scale=..., causal=..., block_table=...)
-> [total_q, Hq, D].  With a block_table, k / v are the KV pools and only the
per-sequence key counts of cu_seqlens_k matter (flash_attn_prefill.py:41-42).
`return_softmax_lse=True` also returns the fp32 [Hq, total_q] log-sum-exp, as
flash_attn_varlen_func does.  There is no host-side scheduler metadata:
fa_version is 0.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


def _int32(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.int32 else t.to(torch.int32)


class FlashAttnPrefill(nn.Module):
    kv_layout = "NHD"

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int):
        super().__init__()
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.sm_scale = head_dim ** -0.5
        self.fa_version = 0
        self._status: torch.Tensor | None = None

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                **kwargs):
        block_table = kwargs.pop("block_table", None)
        scale = kwargs.pop("softmax_scale", None)
        causal = kwargs.pop("causal", True)
        want_lse = bool(kwargs.pop("return_softmax_lse", False))
        window = kwargs.pop("window_size", None)
        if kwargs.pop("s_aux", None) is not None or \
                (window is not None and tuple(window) != (-1, -1)):
            raise NotImplementedError("attention sinks / sliding windows are not on this path")
        for name in ("fa_version", "num_splits", "scheduler_metadata", "seqused_k"):
            kwargs.pop(name, None)
        if kwargs:
            raise TypeError(f"unsupported arguments: {sorted(kwargs)}")
        if self._status is None:
            self._status = ops.new_status(q.device)
        tq = q.shape[0]
        q3 = q.view(tq, self.num_heads, self.head_dim)
        if block_table is None:
            k = k.view(k.shape[0], self.num_kv_heads, self.head_dim)
            v = v.view(v.shape[0], self.num_kv_heads, self.head_dim)
        else:
            block_table = _int32(block_table)
        res = ops.prefill_attn(
            q3, k, v, _int32(cu_seqlens_q), _int32(cu_seqlens_k), int(max_seqlen_q),
            scale if scale is not None else self.sm_scale, causal=causal,
            block_table=block_table, kv_layout=self.kv_layout, return_lse=want_lse,
            status=self._status)
        return res


share_classes(globals())
