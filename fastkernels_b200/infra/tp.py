"""Tensor-parallel rank helpers (mirror of fastkernels/infra/tp.py:8-12)."""
from __future__ import annotations

import torch.distributed as dist


def _tp_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _tp_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
