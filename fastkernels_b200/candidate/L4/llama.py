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


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
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

    def forward(self, input_ids, positions, inputs_embeds=None):
        hidden_states = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
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
