"""KV-cache store (NHD layout).

Drop-in for StoreKVCache (fastkernels/tasks/baseline/L1/store_kvcache.py:71-82):
same class name, same forward(key, value, k_cache, v_cache, slot_mapping) -> None.
The reference casts slot_mapping to int64 on every call (77-78); this kernel
reads int32 or int64 directly, so no cast kernel is launched.
"""
from __future__ import annotations

import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.candidate import share_classes


class StoreKVCache(nn.Module):
    """cache.view(-1, Hkv*D)[slot] = key[i]; rows with slot < 0 are skipped."""

    def forward(self, key, value, k_cache, v_cache, slot_mapping):
        ops.store_kvcache(key, value, k_cache, v_cache, slot_mapping)


class StoreKVCacheHND(nn.Module):
    """HND layout store: [num_blocks, num_kv_heads, block_size, head_dim].
    Drop-in for StoreKVCacheHND (fastkernels/tasks/baseline/L1/store_kvcache.py:85-101)."""

    def __init__(self, page_size: int):
        super().__init__()
        self.page_size = page_size

    def forward(self, key, value, k_cache, v_cache, slot_mapping):
        if k_cache.shape[2] != self.page_size:
            raise ValueError(f"cache page size {k_cache.shape[2]} != {self.page_size}")
        ops.store_kvcache_hnd(key, value, k_cache, v_cache, slot_mapping)


share_classes(globals())
