"""Vocab-parallel embedding and LM head.

Drop-ins for VocabParallelEmbedding / ParallelLMHead
(fastkernels/tasks/baseline/L2/parallel_embedding.py:16-116): the same
constructors and the same methods with the same meaning — masked local lookup +
all-reduce when tp > 1; `project` (the in-graph LM-head GEMM, rows picked by the
step's context as the reference does), `gather_logits`, `gather_greedy(logits)`
and `forward`.  `greedy_pairs` is this build's in-graph form of the greedy path:
it takes the per-row (max, index) pairs the arg-max kernel has already written
and returns the token ids on EVERY rank, so the next step can read them on the
device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from fastkernels_b200 import ops
from fastkernels_b200.infra.context import get_context
from fastkernels_b200.infra.tp import _tp_rank, _tp_size
from fastkernels_b200.candidate.L1.allreduce import AllReduce
from fastkernels_b200.candidate.L1.embedding import Embedding
from fastkernels_b200.candidate.L1.linear import Matmul
from fastkernels_b200.candidate import share_classes


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int,
                 params_dtype: torch.dtype | None = None,
                 org_num_embeddings: int | None = None, padding_size: int = 64):
        super().__init__()
        tp, rank = _tp_size(), _tp_rank()
        assert num_embeddings % tp == 0
        self.num_embeddings = num_embeddings
        self.org_vocab_size = org_num_embeddings or num_embeddings
        self.padding_size = padding_size
        self.embedding_dim = embedding_dim
        self.per_partition = num_embeddings // tp
        self.vocab_start = self.per_partition * rank
        self.vocab_end = self.vocab_start + self.per_partition
        self.tp_size = tp
        self.embedding_op = Embedding(self.per_partition, embedding_dim)
        self.embedding_op.emb.weight.weight_loader = self._weight_loader
        self.allreduce = AllReduce()

    def _weight_loader(self, param, loaded_weight):
        shard = param.data.size(0)
        param.data.copy_(loaded_weight.narrow(0, _tp_rank() * shard, shard))

    def forward(self, x):
        if self.tp_size > 1:
            mask = (x >= self.vocab_start) & (x < self.vocab_end)
            x = mask * (x - self.vocab_start)
        y = self.embedding_op(x)
        if self.tp_size > 1:
            y = mask.unsqueeze(-1) * y
            y = self.allreduce(y)
        return y


class ParallelLMHead(VocabParallelEmbedding):
    def __init__(self, num_embeddings: int, embedding_dim: int, bias: bool = False,
                 params_dtype: torch.dtype | None = None,
                 org_num_embeddings: int | None = None, padding_size: int = 64):
        if bias:
            raise NotImplementedError("ParallelLMHead(bias=True) is not on this path")
        super().__init__(num_embeddings, embedding_dim, params_dtype=params_dtype,
                         org_num_embeddings=org_num_embeddings, padding_size=padding_size)
        self.linear_op = Matmul()

    def project(self, x):
        """LM-head projection only (no gather); runs inside the CUDA graph.  The
        rows are chosen as the reference does (parallel_embedding.py:66-74): all
        of them for decode, each sequence's last token for prefill."""
        ctx = get_context()
        if getattr(ctx, "is_mixed", False):
            x = x[ctx.logit_indices].contiguous()
        elif ctx.is_prefill and ctx.cu_seqlens_q is not None:
            x = x[ctx.cu_seqlens_q[1:].long() - 1].contiguous()
        return self.linear_op(x, self.embedding_op.emb.weight)

    def gather_logits(self, logits):
        """Partial logits of all ranks, concatenated on rank 0 (outside the graph)."""
        if self.tp_size > 1:
            rank = _tp_rank()
            parts = [torch.empty_like(logits) for _ in range(self.tp_size)] if rank == 0 else None
            dist.gather(logits, parts, 0)
            logits = torch.cat(parts, -1) if rank == 0 else logits
        return logits

    def gather_greedy(self, logits):
        """Greedy path of the reference (parallel_embedding.py:83-110): local
        arg-max, all-gather of the (value, global index) pairs, token ids on rank 0
        and None elsewhere; None at tp = 1 (the caller takes the arg-max itself)."""
        if self.tp_size <= 1:
            return None
        if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.dim() == 2:
            vals, idxs = ops.argmax_rows(logits)
        else:
            vals, idxs = logits.max(dim=-1)
        ids = self.greedy_pairs(vals, idxs)
        return ids if _tp_rank() == 0 else None

    def greedy_pairs(self, local_max_vals, local_max_idxs):
        """Token ids from each rank's per-row (max value, LOCAL index): identity at
        tp = 1, else an all-gather of [rows, 2] and the best rank per row; every
        rank gets the ids."""
        if self.tp_size <= 1:
            return local_max_idxs
        info = torch.stack([local_max_vals.float(),
                            (local_max_idxs + self.vocab_start).float()], dim=-1)
        gathered = [torch.empty_like(info) for _ in range(self.tp_size)]
        dist.all_gather(gathered, info)
        all_info = torch.stack(gathered, dim=0)
        best_rank = all_info[:, :, 0].argmax(dim=0)
        rows = torch.arange(info.size(0), device=info.device)
        return all_info[:, :, 1].long()[best_rank, rows]

    def forward(self, x):
        return self.gather_logits(self.project(x))


share_classes(globals())
