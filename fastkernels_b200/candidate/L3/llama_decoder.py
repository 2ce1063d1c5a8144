"""Decoder layer: attention + MLP with fused residual-add RMSNorms.
Drop-in for LlamaDecoderLayer (fastkernels/tasks/baseline/L3/llama_decoder.py:17-42)."""
from __future__ import annotations

import torch.nn as nn

from fastkernels_b200.comm import get_tp_comm
from fastkernels_b200.candidate.L1.rms_norm import RMSNorm
from fastkernels_b200.candidate.L2.attention import LlamaAttention
from fastkernels_b200.candidate.L2.llama_mlp import LlamaMLP
from fastkernels_b200.candidate import share_classes


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config, rotary_emb: nn.Module | None = None, bias: bool = False,
                 qk_norm: bool = False, quant_config: dict | None = None):
        super().__init__()
        self.self_attn = LlamaAttention(
            config.hidden_size, config.num_attention_heads, config.num_key_value_heads,
            config.head_dim, rotary_emb=rotary_emb, bias=bias, qk_norm=qk_norm,
            rms_norm_eps=config.rms_norm_eps, quant_config=quant_config,
            # build-only options: absent from the reference's config, in which case
            # the attention layer follows the engine's backend configuration
            block_size=getattr(config, "kv_block_size", None),
            fused=getattr(config, "fused_attention_prologue", True),
            kv_layout=getattr(config, "kv_layout", None))
        self.mlp = LlamaMLP(config, quant_config=quant_config)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    @staticmethod
    def add_norm(norm: RMSNorm, hidden_states, residual, slot: int):
        """residual-add + RMSNorm; with a tensor-parallel communicator installed,
        `hidden_states` is this rank's un-reduced partial sitting in communication
        slot `slot`, and the all-reduce is fused into the same kernel."""
        comm = get_tp_comm()
        if comm is not None and comm.world > 1:
            rows = hidden_states.shape[0]
            # the fused kernel reads the slot, not `hidden_states`: they must be the
            # same memory (a row-parallel projection without a slot, or one that
            # all-reduced on its own, would leave stale rows there)
            if hidden_states.dim() != 2 or \
                    hidden_states.data_ptr() != comm.slot_view(slot, rows, comm.cols).data_ptr():
                raise RuntimeError("add_norm: hidden_states is not the communication slot "
                                   f"{slot} written by the preceding row-parallel projection")
            return comm.allreduce_add_rmsnorm(slot, rows, residual, norm.weight, norm.eps)
        return norm(hidden_states, residual)

    def forward(self, positions, hidden_states, residual):
        if residual is None:
            hidden_states, residual = self.input_layernorm(hidden_states), hidden_states
        else:
            hidden_states, residual = self.add_norm(self.input_layernorm, hidden_states,
                                                    residual, 1)
        hidden_states = self.self_attn(positions, hidden_states)
        hidden_states, residual = self.add_norm(self.post_attention_layernorm,
                                                hidden_states, residual, 0)
        hidden_states = self.mlp(hidden_states)
        return hidden_states, residual


share_classes(globals())
