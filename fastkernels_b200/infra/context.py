"""Per-step global Context read by the attention layer.

Mirror of the prefill / decode part of fastkernels/infra/context.py: the Context
dataclass fields (172-182), get_context / set_context / reset_context (406-446).
The engine sets it before the model forward (or before graph capture / replay)
and resets it afterwards, exactly as ModelRunner.run does
(fastkernels/infra/engine.py:6057-6063).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Context:
    is_prefill: bool = False
    cu_seqlens_q: torch.Tensor | None = None    # [num_seqs + 1] int32 (prefill)
    cu_seqlens_k: torch.Tensor | None = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: torch.Tensor | None = None    # [N] int32, -1 = padded row
    context_lens: torch.Tensor | None = None    # [N] int32, 0 = padded row
    block_tables: torch.Tensor | None = None    # [N, max_num_blocks] int32, -1 padded
    max_context_len: int = 0
    # set by the engine once it has computed the step's split-KV schedule into the
    # attention workspace all layers share; layers then skip their own plan launch
    attn_plan_ready: bool = False


_CONTEXT = Context()


def get_context() -> Context:
    return _CONTEXT


def set_context(is_prefill, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0,
                max_seqlen_k=0, slot_mapping=None, context_lens=None, block_tables=None,
                max_context_len=0) -> None:
    """Same argument order as the reference's set_context (context.py:411-440,
    the fields this path reads).  Prefill: cu_seqlens / max_seqlen, slot_mapping
    and, when a prefix is already cached, block_tables.  Decode: slot_mapping,
    context_lens, block_tables."""
    global _CONTEXT
    _CONTEXT = Context(bool(is_prefill), cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q),
                       int(max_seqlen_k), slot_mapping, context_lens, block_tables,
                       max_context_len)


def reset_context() -> None:
    global _CONTEXT
    _CONTEXT = Context()
