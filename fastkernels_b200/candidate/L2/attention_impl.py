"""Attention layer: KV store + prefill or paged decode attention.

Drop-in for Attention (fastkernels/tasks/baseline/L2/attention_impl.py:179-450) on
its flash-attn (NHD) and trtllm (HND) paths: the same constructor arguments in
the same order, forward(query, key, value) reads the global Context, stores the
new tokens' K/V and dispatches on ctx.is_prefill exactly as _forward_pure does
(401-450): prefill over the dense k / v of the batch, or over the paged cache
when block tables are given (cached prefix); decode over the paged cache.
`k_cache` / `v_cache` are views the engine installs after allocating the pool
(engine.py:1783-1793).

Features of the reference layer this path does not carry raise at construction
(sliding windows, attention sinks, chunked local attention, the Triton-only
route) or at the call (mixed prefill + decode batches, tree verification); none
of them is used by the Llama / Qwen3 dense decoders.

Page size and pool layout: the two keyword-only arguments win; without them the
layer follows the backend configuration of the reference engine it is running
in (HND / 16 on Blackwell), and outside the reference it defaults to NHD / 256.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200.infra.context import get_context, reference_attn_backend
from fastkernels_b200.candidate.L1.flash_attn_decode import FlashAttnDecode
from fastkernels_b200.candidate.L1.flash_attn_prefill import FlashAttnPrefill
from fastkernels_b200.candidate.L1.flashinfer_decode import TRTLLMDecode
from fastkernels_b200.candidate.L1.flashinfer_prefill import TRTLLMPrefill
from fastkernels_b200.candidate.L1.store_kvcache import StoreKVCache, StoreKVCacheHND
from fastkernels_b200.candidate import share_classes


class Attention(nn.Module):
    def __init__(self, num_heads: int, head_size: int, scale: float,
                 num_kv_heads: int | None = None,
                 sliding_window: int | None = None,
                 sinks: torch.nn.Parameter | None = None,
                 attention_chunk_size: int | None = None,
                 prefer_triton: bool = False,
                 *, block_size: int | None = None, kv_layout: str | None = None):
        super().__init__()
        for name, value in (("sliding_window", sliding_window), ("sinks", sinks),
                            ("attention_chunk_size", attention_chunk_size)):
            if value is not None:
                raise NotImplementedError(f"Attention({name}=...) is not on this path")
        if prefer_triton:
            raise NotImplementedError("Attention(prefer_triton=True) is not on this path")
        self.num_heads = num_heads
        self.head_size = head_size
        self.scale = scale
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.sliding_window = None
        self.sinks = None
        self.attention_chunk_size = None
        self.k_cache = self.v_cache = torch.tensor([])
        if block_size is None or kv_layout is None:
            ref = reference_attn_backend()
            ref_block, ref_layout = ref if ref is not None else (256, "NHD")
            block_size = ref_block if block_size is None else block_size
            kv_layout = ref_layout if kv_layout is None else kv_layout
        if kv_layout not in ("NHD", "HND"):
            raise ValueError("kv_layout must be 'NHD' or 'HND'")
        self._block_size = block_size
        self.kv_layout = kv_layout
        self._use_trtllm = kv_layout == "HND"
        self._triton_only = False
        self._use_custom_op = False
        self._layer_name = ""
        if kv_layout == "HND":      # the reference's trtllm path (attention_impl.py:256-265)
            self.store_kvcache = StoreKVCacheHND(page_size=block_size)
            self.decode_op = TRTLLMDecode(self.num_heads, self.num_kv_heads, head_size)
            self.prefill_op = TRTLLMPrefill(self.num_heads, self.num_kv_heads, head_size)
        else:
            self.store_kvcache = StoreKVCache()
            self.decode_op = FlashAttnDecode(self.num_heads, self.num_kv_heads, head_size,
                                             page_size=block_size)
            self.prefill_op = FlashAttnPrefill(self.num_heads, self.num_kv_heads, head_size)

    def set_trtllm_workspace(self, workspace: torch.Tensor) -> None:
        """The reference engine hands every layer its shared 512 MiB trtllm scratch
        (engine.py:1133-1141); the kernels here do not use it, the reference is
        only kept so that nothing else has to own the buffer."""
        if self._use_trtllm:
            self.decode_op._workspace = workspace
            self.prefill_op._workspace = workspace

    def process_weights_after_loading(self) -> None:
        """Nothing to prepare: there are no attention sinks on this path."""

    def attend(self, q: torch.Tensor, k: torch.Tensor | None = None,
               v: torch.Tensor | None = None) -> torch.Tensor:
        """Attention for q [N, Hq, D] whose K/V are already stored; k / v [N, Hkv, D]
        are the batch's own keys and values, needed for prefill without block
        tables."""
        ctx = get_context()
        if getattr(ctx, "is_mixed", False) or getattr(ctx, "is_tree_verify", False):
            raise NotImplementedError(
                "mixed prefill + decode batches and tree verification are not on this path")
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
                              plan_ready=getattr(ctx, "attn_plan_ready", False))

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


share_classes(globals())
