"""KV-cache store (NHD layout).

Drop-in for StoreKVCache (fastkernels/tasks/baseline/L1/store_kvcache.py:71-82):
same class name, same forward(key, value, k_cache, v_cache, slot_mapping) -> None.
The reference casts slot_mapping to int64 on every call (77-78); this kernel
reads int32 or int64 directly, so no cast kernel is launched.
"""
from __future__ import annotations

import torch.nn as nn

from fastkernels_b200 import ops


class StoreKVCache(nn.Module):
    """cache.view(-1, Hkv*D)[slot] = key[i]; rows with slot < 0 are skipped."""

    def forward(self, key, value, k_cache, v_cache, slot_mapping):
        ops.store_kvcache(key, value, k_cache, v_cache, slot_mapping)
