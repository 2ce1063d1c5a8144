"""torch.library registration of the kernels, so that modules using them can be
traced by torch.compile(fullgraph=True) without graph breaks.

The reference engine compiles the whole model with fullgraph=True unless it runs
with enforce_eager (fastkernels/infra/compilation.py:1665-1671) and its own ops
are registered the same way (fastkernels/tasks/baseline/L1/rms_norm.py:44-69,
fastkernels/tasks/baseline/L1/rotary_emb.py:24-41).  A raw ctypes call is opaque
to Dynamo; these ops give it a schema (with mutation annotations) and a fake
implementation that only describes output shapes.  The candidates route through
them while torch.compiler.is_compiling() and call the C-ABI directly otherwise.
"""
from __future__ import annotations

import torch

from . import ops

_lib = torch.library.Library("fk_b200", "DEF")

_lib.define("rmsnorm(Tensor x, Tensor weight, float eps) -> Tensor")
_lib.define("fused_add_rmsnorm(Tensor(a!) x, Tensor(b!) residual, Tensor weight, float eps) -> ()")
_lib.define("rope_neox(Tensor positions, Tensor(a!) query, Tensor(b!)? key, int head_dim, "
            "Tensor cos_sin_cache) -> ()")
_lib.define("silu_and_mul(Tensor x) -> Tensor")
_lib.define("gemm_bf16(Tensor x, Tensor w, Tensor? bias) -> Tensor")


def _rmsnorm(x, weight, eps):
    return ops.rmsnorm(x, weight, eps)


def _fused_add_rmsnorm(x, residual, weight, eps):
    ops.fused_add_rmsnorm(x, residual, weight, eps)


def _rope_neox(positions, query, key, head_dim, cos_sin_cache):
    ops.rope_neox(positions, query, key, head_dim, cos_sin_cache)


def _silu_and_mul(x):
    return ops.silu_and_mul(x)


def _gemm_bf16(x, w, bias):
    return ops.gemm_bf16(x, w, bias)


_lib.impl("rmsnorm", _rmsnorm, "CUDA")
_lib.impl("fused_add_rmsnorm", _fused_add_rmsnorm, "CUDA")
_lib.impl("rope_neox", _rope_neox, "CUDA")
_lib.impl("silu_and_mul", _silu_and_mul, "CUDA")
_lib.impl("gemm_bf16", _gemm_bf16, "CUDA")


@torch.library.register_fake("fk_b200::rmsnorm")
def _(x, weight, eps):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.register_fake("fk_b200::fused_add_rmsnorm")
def _(x, residual, weight, eps):
    return None


@torch.library.register_fake("fk_b200::rope_neox")
def _(positions, query, key, head_dim, cos_sin_cache):
    return None


@torch.library.register_fake("fk_b200::silu_and_mul")
def _(x):
    return torch.empty((*x.shape[:-1], x.shape[-1] // 2), dtype=x.dtype, device=x.device)


@torch.library.register_fake("fk_b200::gemm_bf16")
def _(x, w, bias):
    return torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
