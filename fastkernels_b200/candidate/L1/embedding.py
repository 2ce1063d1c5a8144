"""Token embedding.  Mirror of Embedding
(fastkernels/tasks/baseline/L1/embedding.py): a gather, kept on nn.Embedding."""
from __future__ import annotations

import torch.nn as nn


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.emb = nn.Embedding(num_embeddings, embedding_dim)

    def forward(self, x):
        return self.emb(x)
