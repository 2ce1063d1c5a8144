"""Per-step global Context read by the attention layer.

Mirror of the prefill / decode part of fastkernels/infra/context.py: the Context
dataclass fields (172-182), get_context / set_context / reset_context (406-446).
The engine sets it before the model forward (or before graph capture / replay)
and resets it afterwards, exactly as ModelRunner.run does
(fastkernels/infra/engine.py:6057-6063).

Inside the reference's own serving engine it is the reference's context module
that gets set (fastkernels/infra/engine.py:6057-6063 calls
fastkernels.infra.context.set_context), so get_context() here hands out THAT
object whenever this package's own set_context has not been called and the
reference module is loaded: the swapped-in candidates then read what the engine
wrote.  The field names this path reads are the same in both dataclasses.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass

import torch

_REFERENCE_CONTEXT_MODULE = "fastkernels.infra.context"


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
_OWN_CONTEXT_SET = False


def get_context():
    """This package's context while its own engine has one set; otherwise the
    reference engine's context when that module is loaded; otherwise the empty
    default."""
    if not _OWN_CONTEXT_SET:
        ref = sys.modules.get(_REFERENCE_CONTEXT_MODULE)
        if ref is not None:
            return ref.get_context()
    return _CONTEXT


def reference_attn_backend():
    """(block_size, kv_layout) the reference engine will allocate its KV pool
    with (AttnBackendConfig, fastkernels/infra/context.py:28-75: HND / 16 on
    Blackwell when FlashInfer's trtllm decode imports, else NHD), or None when the
    reference package is not loaded."""
    ref = sys.modules.get(_REFERENCE_CONTEXT_MODULE)
    if ref is None:
        return None
    cfg = ref.get_attn_backend_config()
    return int(cfg.block_size), ("HND" if cfg.use_trtllm else "NHD")


def set_context(is_prefill, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0,
                max_seqlen_k=0, slot_mapping=None, context_lens=None, block_tables=None,
                max_context_len=0) -> None:
    """Same argument order as the reference's set_context (context.py:411-440,
    the fields this path reads).  Prefill: cu_seqlens / max_seqlen, slot_mapping
    and, when a prefix is already cached, block_tables.  Decode: slot_mapping,
    context_lens, block_tables."""
    global _CONTEXT, _OWN_CONTEXT_SET
    _OWN_CONTEXT_SET = True
    _CONTEXT = Context(bool(is_prefill), cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q),
                       int(max_seqlen_k), slot_mapping, context_lens, block_tables,
                       max_context_len)


def reset_context() -> None:
    global _CONTEXT, _OWN_CONTEXT_SET
    _OWN_CONTEXT_SET = False
    _CONTEXT = Context()
