"""Model-level attention block: qkv_proj -> [q/k norm] -> RoPE -> store + decode
attention -> o_proj.

Drop-in for LlamaAttention (fastkernels/tasks/baseline/L2/attention.py:29-156)
for the Llama / Qwen3 dense prefill and decode paths (bias, qk_norm options): the
same constructor arguments in the same order; the Llama-4 and GPT-OSS options
(nope, weight-less q/k norm, temperature tuning, chunked attention, sinks,
sliding window) and fp8 weights raise when asked for.  With `fused=True`
(default) the split, per-head q/k RMSNorm, RoPE and KV store run as ONE kernel
over the packed qkv rows (fk_qkv_rope_store); `fused=False` runs the reference's
op-by-op chain on the L1 drop-ins.  `block_size` / `kv_layout` default to the
backend configuration of the engine the layer is built in (see Attention).
"""
from __future__ import annotations

import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes
from fastkernels_b200.infra.context import get_context
from fastkernels_b200.infra.tp import _tp_size
from fastkernels_b200.candidate.L1.rms_norm import RMSNorm
from fastkernels_b200.candidate.L2.attention_impl import Attention
from fastkernels_b200.candidate.L2.parallel_linear import QKVParallelLinear, RowParallelLinear


class LlamaAttention(nn.Module):
    def __init__(self, hidden_size: int, num_attention_heads: int, num_key_value_heads: int,
                 head_dim: int, rotary_emb: nn.Module | None = None, bias: bool = False,
                 qk_norm: bool = False, rms_norm_eps: float = 1e-6,
                 nope: bool = False, use_weightless_qk_norm: bool = False,
                 attn_temperature_tuning: bool = False, floor_scale: float = 8192.0,
                 attn_scale: float = 0.1, quant_config: dict | None = None,
                 attention_chunk_size: int | None = None, o_proj_bias: bool = False,
                 use_sinks: bool = False, sliding_window: int | None = None,
                 layer_idx: int = 0,
                 *, block_size: int | None = None, fused: bool = True,
                 kv_layout: str | None = None):
        super().__init__()
        unsupported = dict(nope=nope, use_weightless_qk_norm=use_weightless_qk_norm,
                           attn_temperature_tuning=attn_temperature_tuning,
                           quant_config=quant_config is not None,
                           attention_chunk_size=attention_chunk_size is not None,
                           use_sinks=use_sinks,
                           # the reference applies the window on even layers only
                           sliding_window=sliding_window is not None and layer_idx % 2 == 0)
        asked = [k for k, v in unsupported.items() if v]
        if asked:
            raise NotImplementedError(f"LlamaAttention({', '.join(asked)}) is not on this path")
        tp = _tp_size()
        self.num_heads = num_attention_heads // tp
        self.num_kv_heads = num_key_value_heads // tp if num_key_value_heads >= tp else 1
        self.head_dim = head_dim
        self.rotary_emb = rotary_emb
        self.rms_norm_eps = rms_norm_eps
        self.nope = False
        self.attn_temperature_tuning = False
        self.floor_scale, self.attn_scale = floor_scale, attn_scale
        self.sinks = None
        self.fused = fused
        self.qkv_proj = QKVParallelLinear(hidden_size, head_dim, num_attention_heads,
                                          num_key_value_heads, bias=bias)
        self.o_proj = RowParallelLinear(num_attention_heads * head_dim, hidden_size,
                                        bias=o_proj_bias)
        self.o_proj.comm_slot = 0
        self.q_norm = RMSNorm(head_dim, eps=rms_norm_eps) if qk_norm else None
        self.k_norm = RMSNorm(head_dim, eps=rms_norm_eps) if qk_norm else None
        self.q_wl_norm = self.k_wl_norm = None
        self.attn = Attention(self.num_heads, head_dim, head_dim ** -0.5,
                              num_kv_heads=self.num_kv_heads, block_size=block_size,
                              kv_layout=kv_layout)

    def forward(self, positions, hidden_states, rotary_emb=None):
        n = hidden_states.shape[0]
        qkv = self.qkv_proj(hidden_states)
        q_size = self.num_heads * self.head_dim
        kv_size = self.num_kv_heads * self.head_dim
        rope = rotary_emb if rotary_emb is not None else self.rotary_emb
        if self.fused and rope is not None and self.attn.k_cache.numel() \
                and hasattr(rope, "activation_cache"):
            ctx = get_context()
            ops.qkv_rope_store(
                qkv, self.num_heads, self.num_kv_heads, self.head_dim, positions,
                rope.activation_cache(qkv.dtype, qkv.device),
                self.q_norm.weight if self.q_norm is not None else None,
                self.k_norm.weight if self.k_norm is not None else None,
                self.rms_norm_eps, self.attn.k_cache, self.attn.v_cache, ctx.slot_mapping,
                kv_layout=self.attn.kv_layout)
            q = qkv[:, :q_size].view(n, self.num_heads, self.head_dim)
            k = qkv[:, q_size:q_size + kv_size].view(n, self.num_kv_heads, self.head_dim)
            v = qkv[:, q_size + kv_size:].view(n, self.num_kv_heads, self.head_dim)
            o = self.attn.attend(q, k, v).reshape(n, q_size)
            return self.o_proj(o)
        q, k, v = qkv.split([q_size, kv_size, kv_size], dim=-1)
        if self.q_norm is not None:
            q_shape, k_shape = q.shape, k.shape
            q = self.q_norm(q.view(n, self.num_heads, self.head_dim)).view(q_shape)
            k = self.k_norm(k.view(n, self.num_kv_heads, self.head_dim)).view(k_shape)
        if rope is not None:
            q, k = rope(positions, q, k)
        return self.o_proj(self.attn(q, k, v))


share_classes(globals())
