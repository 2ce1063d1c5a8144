"""Tensor-parallel linear layers on the tcgen05 decode GEMM.

Drop-ins for ColumnParallelLinear / MergedColumnParallelLinear /
QKVParallelLinear / RowParallelLinear
(fastkernels/tasks/baseline/L2/parallel_linear.py:33-335, bf16 path): same
constructors, parameter names and shard layout, same weight_loader semantics
(column shards along dim 0, row shards along dim 1, merged gate/up and q/k/v
blocks sharded independently), RowParallelLinear adds the bias on rank 0 only
and all-reduces when tp > 1.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.comm import get_tp_comm
from fastkernels_b200.infra.tp import _tp_rank, _tp_size
from fastkernels_b200.candidate.L1.allreduce import AllReduce
from fastkernels_b200.candidate import share_classes


def _linear(x, weight, bias):
    shape = x.shape
    if torch.compiler.is_compiling():
        import fastkernels_b200.torch_ops  # noqa: F401  (registers fk_b200::*)
        y = torch.ops.fk_b200.gemm_bf16(x.reshape(-1, shape[-1]), weight, bias)
    else:
        y = ops.gemm_bf16(x.reshape(-1, shape[-1]), weight, bias)
    return y.view(*shape[:-1], weight.shape[0])


class ColumnParallelLinear(nn.Module):
    """Splits the output dim across TP ranks."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 quant_config: dict | None = None):
        super().__init__()
        if quant_config is not None:
            raise NotImplementedError("fp8 weights are not on this path")
        tp = _tp_size()
        assert output_size % tp == 0
        self.output_size_per_partition = output_size // tp
        self.weight = nn.Parameter(torch.empty(self.output_size_per_partition, input_size))
        self.weight.weight_loader = self._weight_loader
        self.bias = nn.Parameter(torch.empty(self.output_size_per_partition)) if bias else None
        if self.bias is not None:
            self.bias.weight_loader = self._weight_loader

    def _weight_loader(self, param, loaded_weight):
        shard = param.data.size(0)
        param.data.copy_(loaded_weight.narrow(0, _tp_rank() * shard, shard))

    def forward(self, x):
        return _linear(x, self.weight, self.bias)


class MergedColumnParallelLinear(nn.Module):
    """gate_proj + up_proj merged into one linear, each block sharded across TP."""

    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False,
                 quant_config: dict | None = None, disable_tp: bool = False):
        super().__init__()
        if quant_config is not None:
            raise NotImplementedError("fp8 weights are not on this path")
        tp = 1 if disable_tp else _tp_size()
        self.disable_tp = disable_tp
        self.output_sizes = output_sizes
        assert all(s % tp == 0 for s in output_sizes)
        total = sum(output_sizes)
        self.weight = nn.Parameter(torch.empty(total // tp, input_size))
        self.weight.weight_loader = self._weight_loader
        self.bias = None
        if bias:
            self.bias = nn.Parameter(torch.empty(total // tp))
            self.bias.weight_loader = self._weight_loader

    def _weight_loader(self, param, loaded_weight, shard_id: int | None = None):
        tp = 1 if self.disable_tp else _tp_size()
        if shard_id is None:
            offset = 0
            for sid, sz in enumerate(self.output_sizes):
                self._weight_loader(param, loaded_weight.narrow(0, offset, sz), sid)
                offset += sz
            return
        shard_offset = sum(self.output_sizes[:shard_id]) // tp
        shard_size = self.output_sizes[shard_id] // tp
        dst = param.data.narrow(0, shard_offset, shard_size)
        dst.copy_(loaded_weight if tp == 1 else loaded_weight.chunk(tp, 0)[_tp_rank()])

    def forward(self, x):
        return _linear(x, self.weight, self.bias)


class QKVParallelLinear(nn.Module):
    """Q, K, V projections merged and sharded by heads across TP."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int,
                 total_num_kv_heads: int, bias: bool = False,
                 quant_config: dict | None = None):
        super().__init__()
        if quant_config is not None:
            raise NotImplementedError("fp8 weights are not on this path")
        tp = _tp_size()
        self.head_size = head_size
        self.num_heads = total_num_heads // tp
        if total_num_kv_heads % tp == 0:
            self.num_kv_heads = total_num_kv_heads // tp
            self._replicate_kv = False
        else:
            self.num_kv_heads = total_num_kv_heads
            self._replicate_kv = True
        output_size = (self.num_heads + 2 * self.num_kv_heads) * head_size
        self.weight = nn.Parameter(torch.empty(output_size, hidden_size))
        self.weight.weight_loader = self._weight_loader
        self.bias = None
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size))
            self.bias.weight_loader = self._weight_loader

    def _weight_loader(self, param, loaded_weight, shard_id: str):
        tp, rank = _tp_size(), _tp_rank()
        q_size = self.num_heads * self.head_size
        kv_size = self.num_kv_heads * self.head_size
        if shard_id == "q":
            size, offset = q_size, 0
            src = loaded_weight.chunk(tp, 0)[rank]
        else:
            size = kv_size
            offset = q_size if shard_id == "k" else q_size + kv_size
            src = loaded_weight if self._replicate_kv else loaded_weight.chunk(tp, 0)[rank]
        param.data.narrow(0, offset, size).copy_(src)

    def forward(self, x):
        return _linear(x, self.weight, self.bias)


class RowParallelLinear(nn.Module):
    """Splits the input dim across TP ranks and all-reduces the output."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False,
                 quant_config: dict | None = None, reduce_results: bool = True):
        super().__init__()
        if quant_config is not None:
            raise NotImplementedError("fp8 weights are not on this path")
        tp = _tp_size()
        assert input_size % tp == 0
        self.input_size_per_partition = input_size // tp
        self.tp_size = tp
        self.tp_rank = _tp_rank()
        self.reduce_results = reduce_results
        self.weight = nn.Parameter(torch.empty(output_size, self.input_size_per_partition))
        self.weight.weight_loader = self._weight_loader
        self.bias = nn.Parameter(torch.empty(output_size)) if bias else None
        if self.bias is not None:
            self.bias.weight_loader = lambda p, w: p.data.copy_(w)
        self.allreduce = AllReduce()
        # set by the enclosing block when its output feeds a fused
        # all-reduce + add + RMSNorm: which communication slot to write into
        self.comm_slot: int | None = None

    def _weight_loader(self, param, loaded_weight):
        shard = param.data.size(1)
        param.data.copy_(loaded_weight.narrow(1, _tp_rank() * shard, shard))

    def forward(self, x):
        bias = self.bias if self.tp_rank == 0 else None
        comm = get_tp_comm()
        if (comm is not None and self.comm_slot is not None and self.reduce_results
                and self.tp_size > 1 and x.dim() == 2):
            # un-reduced partial, written straight into the communication slot; the
            # norm that follows reduces it across ranks (fk_allreduce_add_rmsnorm)
            if comm.pushed(x.shape[0]):
                # the projection's tiles go straight into every rank's receive area
                return comm.gemm_push(x, self.weight, bias, self.comm_slot)
            out = comm.slot_view(self.comm_slot, x.shape[0], self.weight.shape[0])
            return ops.gemm_bf16(x, self.weight, bias, out=out)
        y = _linear(x, self.weight, bias)
        if self.reduce_results and self.tp_size > 1:
            y = self.allreduce(y)
        return y


share_classes(globals())
