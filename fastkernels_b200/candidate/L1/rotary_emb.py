"""NeoX rotary position embedding, in place.

Drop-in for RotaryEmbedding (fastkernels/tasks/baseline/L1/rotary_emb.py:70-191):
same constructor (incl. the Llama-3.1 frequency scaling, 44-67), the same
non-persistent fp32 buffer `cos_sin_cache` [max_pos, head_dim] = cat(cos, sin),
forward(positions, query, key) -> (query, key) rotated in place.

The reference casts the whole fp32 cache to the activation dtype on every call
(171-173); here the rounded copy is made once and reused.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


def _compute_scaled_inv_freq(inv_freq, scaling_factor, low_freq_factor, high_freq_factor,
                             original_max_position_embeddings):
    low_wl = original_max_position_embeddings / low_freq_factor
    high_wl = original_max_position_embeddings / high_freq_factor
    wl = 2 * math.pi / inv_freq
    if low_freq_factor != high_freq_factor:
        smooth = (original_max_position_embeddings / wl - low_freq_factor) / (
            high_freq_factor - low_freq_factor)
    else:
        smooth = torch.zeros_like(inv_freq)
    return torch.where(
        wl < high_wl, inv_freq,
        torch.where(wl > low_wl, inv_freq / scaling_factor,
                    (1 - smooth) * inv_freq / scaling_factor + smooth * inv_freq))


class RotaryEmbedding(nn.Module):
    def __init__(self, head_dim: int, max_position_embeddings: int, rope_theta: float,
                 rope_scaling_factor: float = 1.0, rope_low_freq_factor: float = 1.0,
                 rope_high_freq_factor: float = 1.0,
                 rope_original_max_position_embeddings: int | None = None,
                 is_neox_style: bool = True):
        super().__init__()
        if not is_neox_style:
            raise NotImplementedError("only the NeoX pairing is on the decode path")
        self.head_dim = head_dim
        self.is_neox_style = True
        inv_freq = 1.0 / (rope_theta ** (
            torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
        if rope_scaling_factor != 1.0 and rope_original_max_position_embeddings is not None:
            inv_freq = _compute_scaled_inv_freq(
                inv_freq, rope_scaling_factor, rope_low_freq_factor, rope_high_freq_factor,
                rope_original_max_position_embeddings)
        t = torch.arange(max_position_embeddings, dtype=torch.float)
        freqs = torch.einsum("i,j -> ij", t, inv_freq)
        cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1).float()
        self.register_buffer("cos_sin_cache", cache, persistent=False)
        self._cache_act: torch.Tensor | None = None

    def activation_cache(self, dtype, device) -> torch.Tensor:
        """cos_sin_cache rounded to the activation dtype, made once."""
        c = self._cache_act
        if c is None or c.dtype != dtype or c.device != torch.device(device):
            c = self.cos_sin_cache.to(device=device, dtype=dtype)
            self._cache_act = c
        return c

    def forward(self, positions, query, key):
        if torch.compiler.is_compiling():
            import fastkernels_b200.torch_ops  # noqa: F401  (registers fk_b200::*)
            # the fp32 buffer is rounded to bf16 inside the kernel: no cached copy
            # to create while tracing
            torch.ops.fk_b200.rope_neox(positions, query, key, self.head_dim,
                                        self.cos_sin_cache)
            return query, key
        cache = self.activation_cache(query.dtype, query.device)
        ops.rope_neox(positions, query, key, self.head_dim, cache)
        return query, key


share_classes(globals())
