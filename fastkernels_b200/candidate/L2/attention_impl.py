"""Attention layer: KV store + prefill or paged decode attention.

Mirror of Attention (fastkernels/tasks/baseline/L2/attention_impl.py:179-450) on
its flash-attn (NHD) and trtllm (HND) paths: forward(query, key, value) reads the
global Context, stores the new tokens' K/V and dispatches on ctx.is_prefill
exactly as _forward_pure does (401-450): prefill over the dense k / v of the
batch, or over the paged cache when block tables are given (cached prefix);
decode over the paged cache.  `k_cache` / `v_cache` are
views the engine installs after allocating the pool (engine.py:1783-1793).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200.infra.context import get_context
from fastkernels_b200.candidate.L1.flash_attn_decode import FlashAttnDecode
from fastkernels_b200.candidate.L1.flash_attn_prefill import FlashAttnPrefill
from fastkernels_b200.candidate.L1.flashinfer_decode import TRTLLMDecode
from fastkernels_b200.candidate.L1.flashinfer_prefill import TRTLLMPrefill
from fastkernels_b200.candidate.L1.store_kvcache import StoreKVCache, StoreKVCacheHND


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_size: int, scale: float,
                 num_kv_heads: int | None = None, block_size: int = 256,
                 kv_layout: str = "NHD"):
        super().__init__()
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = scale
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.k_cache = self.v_cache = torch.tensor([])
        self._block_size = block_size
        self.kv_layout = kv_layout
        if kv_layout == "HND":      # the reference's trtllm path (attention_impl.py:256-265)
            self.store_kvcache = StoreKVCacheHND(page_size=block_size)
            self.decode_op = TRTLLMDecode(self.num_heads, self.num_kv_heads, head_size)
            self.prefill_op = TRTLLMPrefill(self.num_heads, self.num_kv_heads, head_size)
        else:
            self.store_kvcache = StoreKVCache()
            self.decode_op = FlashAttnDecode(self.num_heads, self.num_kv_heads, head_size,
                                             page_size=block_size)
            self.prefill_op = FlashAttnPrefill(self.num_heads, self.num_kv_heads, head_size)

    def attend(self, q: torch.Tensor, k: torch.Tensor | None = None,
               v: torch.Tensor | None = None) -> torch.Tensor:
        """Attention for q [N, Hq, D] whose K/V are already stored; k / v [N, Hkv, D]
        are the batch's own keys and values, needed for prefill without block
        tables."""
        ctx = get_context()
        if ctx.is_prefill:
            kw = dict(cu_seqlens_q=ctx.cu_seqlens_q, cu_seqlens_k=ctx.cu_seqlens_k,
                      max_seqlen_q=ctx.max_seqlen_q, max_seqlen_k=ctx.max_seqlen_k,
                      softmax_scale=self.scale, causal=True)
            if ctx.block_tables is not None:
                return self.prefill_op(q, self.k_cache, self.v_cache,
                                       block_table=ctx.block_tables, **kw)
            return self.prefill_op(q, k, v, **kw)
        return self.decode_op(q, self.k_cache, self.v_cache,
                              cache_seqlens=ctx.context_lens, block_table=ctx.block_tables,
                              softmax_scale=self.scale, causal=True,
                              max_seq_len=ctx.max_context_len,
                              plan_ready=ctx.attn_plan_ready)

    def decode_only(self, q: torch.Tensor) -> torch.Tensor:
        return self.attend(q)

    def forward_impl(self, query, key, value):
        ctx = get_context()
        n = query.shape[0]
        q = query.view(n, self.num_heads, self.head_size)
        k = key.view(n, self.num_kv_heads, self.head_size)
        v = value.view(n, self.num_kv_heads, self.head_size)
        if self.k_cache.numel() and self.v_cache.numel():
            self.store_kvcache(k, v, self.k_cache, self.v_cache, ctx.slot_mapping)
        o = self.attend(q, k, v)
        return o.reshape(n, self.num_heads * self.head_size)

    def forward(self, query, key, value):
        return self.forward_impl(query, key, value)
