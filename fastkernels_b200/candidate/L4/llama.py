"""Llama / Qwen3-style dense decoder for the decode step.

Mirror of LlamaConfig / LlamaModel / LlamaForCausalLM
(fastkernels/tasks/baseline/L4/llama.py:24-175).  One addition: `qk_norm` in the
config builds the Qwen3 stack (per-head q/k RMSNorm before RoPE), which the
reference assembles as LlamaDecoderLayer(config, rotary_emb=..., qk_norm=True)
(fastkernels/tasks/baseline/L4/qwen3_vl.py:248-251).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.infra.context import get_context
from fastkernels_b200.infra.tp import _tp_size
from fastkernels_b200.candidate.L1.rms_norm import RMSNorm
from fastkernels_b200.candidate.L1.rotary_emb import RotaryEmbedding
from fastkernels_b200.candidate.L2.parallel_embedding import (ParallelLMHead,
                                                               VocabParallelEmbedding)
from fastkernels_b200.candidate.L3.llama_decoder import LlamaDecoderLayer
from fastkernels_b200.candidate import share_classes

__targets__ = ["LlamaForCausalLM"]


@dataclass
class LlamaConfig:
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 128256
    max_position_embeddings: int = 131072
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling_factor: float = 1.0
    rope_low_freq_factor: float = 1.0
    rope_high_freq_factor: float = 1.0
    rope_original_max_position_embeddings: int = 8192
    dtype: torch.dtype = torch.bfloat16
    qkv_bias: bool = False
    qk_norm: bool = False
    kv_block_size: int = 256
    kv_layout: str = "NHD"     # "HND" = the reference's B200 default (page size 16)
    fused_attention_prologue: bool = True
    # decode batches of up to 128 rows on one GPU: run everything between two
    # attention calls as one persistent kernel (fk_decode_block).  Off by default:
    # measured on B200 the one-kernel-per-op chain is the faster of the two today
    decode_block: bool = False


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size)
        self.rotary_emb = RotaryEmbedding(
            config.head_dim, config.max_position_embeddings, config.rope_theta,
            rope_scaling_factor=config.rope_scaling_factor,
            rope_low_freq_factor=config.rope_low_freq_factor,
            rope_high_freq_factor=config.rope_high_freq_factor,
            rope_original_max_position_embeddings=config.rope_original_max_position_embeddings)
        self.layers = nn.ModuleList([
            LlamaDecoderLayer(config, rotary_emb=self.rotary_emb, bias=config.qkv_bias,
                              qk_norm=getattr(config, "qk_norm", False))
            for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def _block_path(self, hidden_states) -> bool:
        """The persistent-block path serves plain decode steps on one GPU."""
        cfg = self.config
        if not getattr(cfg, "decode_block", False) or torch.compiler.is_compiling():
            return False
        if _tp_size() != 1 or not hidden_states.is_cuda or hidden_states.dim() != 2:
            return False
        if hidden_states.dtype != torch.bfloat16 or cfg.head_dim != 128:
            return False
        if hidden_states.shape[0] > ops.decode_block_max_rows() or get_context().is_prefill:
            return False
        first = self.layers[0]
        return bool(first.self_attn.attn.k_cache.numel()) and \
            hasattr(self.rotary_emb, "activation_cache") and first.self_attn.fused and \
            cfg.intermediate_size % 64 == 0 and cfg.hidden_size % 64 == 0

    def _forward_blocks(self, hidden_states, positions):
        """LlamaModel.forward (fastkernels/tasks/baseline/L4/llama.py:100-116) with the
        kernels between two attention calls grouped into one launch each:
          [input norm, qkv projection, split + q/k norm + RoPE + KV store]   layer 0
          attention
          [o projection, add + norm, gate/up + SiLU, down projection,
           add + next layer's input norm, its qkv projection, its RoPE + store]
          attention ... and after the last layer [..., down projection, add + final norm].
        The composition and every rounding point are those of the layer-by-layer path."""
        ctx = get_context()
        m = hidden_states.shape[0]
        dev = hidden_states.device
        cache = self.rotary_emb.activation_cache(hidden_states.dtype, dev)
        residual = hidden_states           # layer 0: residual = embeddings (llama_decoder.py:35-36)

        def attention_prologue(prog, layer, x):
            att = layer.self_attn
            qkv = prog.gemm(x, att.qkv_proj.weight, att.qkv_proj.bias)
            prog.qkv_rope_store(
                qkv, att.num_heads, att.num_kv_heads, att.head_dim, positions, cache,
                att.q_norm.weight if att.q_norm is not None else None,
                att.k_norm.weight if att.k_norm is not None else None,
                att.rms_norm_eps, att.attn.k_cache, att.attn.v_cache, ctx.slot_mapping,
                kv_layout=att.attn.kv_layout)
            return qkv

        prog = ops.BlockProgram(m, dev)
        first = self.layers[0]
        x = prog.add_rmsnorm(None, residual, first.input_layernorm.weight,
                             first.input_layernorm.eps)
        qkv = attention_prologue(prog, first, x)
        prog.launch()
        out = None
        for li, layer in enumerate(self.layers):
            att = layer.self_attn
            q_size, kv_size = att.num_heads * att.head_dim, att.num_kv_heads * att.head_dim
            q = qkv[:, :q_size].view(m, att.num_heads, att.head_dim)
            k = qkv[:, q_size:q_size + kv_size].view(m, att.num_kv_heads, att.head_dim)
            v = qkv[:, q_size + kv_size:].view(m, att.num_kv_heads, att.head_dim)
            o = att.attn.attend(q, k, v).reshape(m, q_size)
            prog = ops.BlockProgram(m, dev)
            y = prog.gemm(o, att.o_proj.weight, att.o_proj.bias)
            x = prog.add_rmsnorm(y, residual, layer.post_attention_layernorm.weight,
                                 layer.post_attention_layernorm.eps)
            mlp = layer.mlp
            act = prog.gemm_silu_mul(x, mlp.gate_up_proj.weight, mlp.gate_up_proj.bias)
            y = prog.gemm(act, mlp.down_proj.weight, mlp.down_proj.bias)
            if li + 1 < len(self.layers):
                nxt = self.layers[li + 1]
                x = prog.add_rmsnorm(y, residual, nxt.input_layernorm.weight,
                                     nxt.input_layernorm.eps)
                qkv = attention_prologue(prog, nxt, x)
            else:
                out = prog.add_rmsnorm(y, residual, self.norm.weight, self.norm.eps)
            prog.launch()
        return out

    def forward(self, input_ids, positions, inputs_embeds=None):
        hidden_states = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        if self._block_path(hidden_states):
            return self._forward_blocks(hidden_states, positions)
        residual = None
        for layer in self.layers:
            hidden_states, residual = layer(positions, hidden_states, residual)
        hidden_states, _ = LlamaDecoderLayer.add_norm(self.norm, hidden_states, residual, 1)
        return hidden_states


class LlamaForCausalLM(nn.Module):
    # checkpoint name -> (merged parameter, shard id), read by the reference's
    # weight loader (fastkernels/tasks/baseline/L4/llama.py:120-126)
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"),
        "k_proj": ("qkv_proj", "k"),
        "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0),
        "up_proj": ("gate_up_proj", 1),
    }

    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size)

    def forward(self, input_ids, positions):
        return self.model(input_ids, positions)

    def forward_with_lm_proj(self, input_ids, positions):
        return self.lm_head.project(self.model(input_ids, positions))

    def set_eagle3_layers_to_capture(self, layer_ids=None):
        raise NotImplementedError("EAGLE-3 hidden-state capture is not on this path")

    # the three sampling-side entry points of the reference model
    # (fastkernels/tasks/baseline/L4/llama.py:157-175)
    def compute_logits(self, hidden_states):
        logits = self.lm_head(hidden_states)
        return logits.float() if logits is not None else None

    def compute_logits_decode(self, partial_logits):
        logits = self.lm_head.gather_logits(partial_logits)
        return logits.float() if logits is not None else None

    def greedy_sample_decode(self, partial_logits):
        return self.lm_head.gather_greedy(partial_logits.float())


share_classes(globals())
