"""Paged GQA decode attention.

Drop-in for FlashAttnDecode (fastkernels/tasks/baseline/L1/flash_attn_decode.py:
22-181): same constructor, same forward(q, k_cache, v_cache, cache_seqlens,
block_table=..., softmax_scale=..., causal=..., max_seq_len=...) -> [N, Hq, D],
and the duck-typed surface the engine touches (preallocate,
update_scheduler_metadata, fa_version, _window_size, _cu_seqlens_q, _sched_buf,
_sched_meta; fastkernels/infra/engine.py:1526-1550).

`causal` is accepted and has no effect: every sequence brings ONE query token,
which sits at the end of its context, so the bottom-right-aligned causal mask the
reference asks for (flash_attn_decode.py:164-181, max_seqlen_q = 1) and no mask at
all select the same keys.

The split-KV schedule is computed on the device from cache_seqlens inside the
call, so there is no host-side scheduler metadata to refresh between graph
replays: update_scheduler_metadata is a no-op and fa_version is 0.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class FlashAttnDecode(nn.Module):
    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int,
                 page_size: int | None = None):
        super().__init__()
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.page_size = page_size
        self.fa_version = 0
        self._cu_seqlens_q = None
        self._sched_buf = None
        self._sched_meta = None
        self._window_size = (-1, -1)
        self._qkv_dtype = torch.bfloat16
        self._workspace: torch.Tensor | None = None
        self._ws_batch = 0
        self._max_splits = 32
        self._status: torch.Tensor | None = None

    def update_scheduler_metadata(self, cache_seqlens, max_seqlen_k, qkv_dtype=None,
                                  window_size=(-1, -1), max_seqlen_q=1) -> None:
        self._sched_meta = None

    def _ensure_workspace(self, batch: int, device) -> None:
        if self._workspace is not None and self._ws_batch >= batch and \
                self._workspace.device == torch.device(device):
            return
        n = ops.attn_workspace_bytes(batch, self.num_heads, self.head_dim, self._max_splits)
        self._workspace = torch.empty(n, dtype=torch.uint8, device=device)
        self._ws_batch = batch
        if self._status is None:
            self._status = ops.new_status(device)

    def preallocate(self, max_batch_size: int, device) -> None:
        """Allocate the graph-stable split-KV workspace before capture."""
        self._ensure_workspace(max_batch_size, device)

    def forward(self, q, k_cache, v_cache, cache_seqlens=None, **kwargs):
        block_table = kwargs.pop("block_table", None)
        softmax_scale = kwargs.pop("softmax_scale", None)
        kwargs.pop("causal", None)
        kwargs.pop("max_seq_len", None)
        planned = bool(kwargs.pop("plan_ready", False))
        window = kwargs.pop("window_size", self._window_size)
        if kwargs.pop("s_aux", None) is not None or tuple(window) != (-1, -1):
            raise NotImplementedError("attention sinks / sliding windows are not on this path")
        if softmax_scale is None:
            softmax_scale = self.head_dim ** -0.5
        self._ensure_workspace(q.shape[0], q.device)
        return ops.paged_decode_attn(q, k_cache, v_cache, cache_seqlens, block_table,
                                     softmax_scale, self._workspace, self._max_splits,
                                     status=self._status, planned=planned)


share_classes(globals())
