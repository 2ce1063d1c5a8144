"""Vocab-parallel embedding and LM head.

Mirrors VocabParallelEmbedding / ParallelLMHead
(fastkernels/tasks/baseline/L2/parallel_embedding.py:16-116) for decode: masked
local lookup + all-reduce when tp > 1; `project` is the in-graph LM-head GEMM,
`gather_greedy` the (max, index) all-gather of the greedy path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from fastkernels_b200.infra.tp import _tp_rank, _tp_size
from fastkernels_b200.candidate.L1.allreduce import AllReduce
from fastkernels_b200.candidate.L1.embedding import Embedding
from fastkernels_b200.candidate.L1.linear import Matmul


class VocabParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        tp, rank = _tp_size(), _tp_rank()
        assert num_embeddings % tp == 0
        self.num_embeddings = num_embeddings
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
    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__(num_embeddings, embedding_dim)
        self.linear_op = Matmul()

    def project(self, x):
        """LM-head projection of the decode rows (no gather); runs in the graph."""
        return self.linear_op(x, self.embedding_op.emb.weight)

    def gather_greedy(self, local_max_vals, local_max_idxs):
        """tp > 1: all-gather each rank's (max value, global index) pair and take
        the best rank per row (parallel_embedding.py:83-110); every rank gets
        the token ids."""
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
