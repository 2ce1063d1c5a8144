"""Token embedding.  Mirror of Embedding
(fastkernels/tasks/baseline/L1/embedding.py): a gather, kept on nn.Embedding."""
from __future__ import annotations

import torch.nn as nn
from fastkernels_b200.candidate import share_classes


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int,
                 padding_idx: int | None = None):
        super().__init__()
        self.emb = nn.Embedding(num_embeddings, embedding_dim, padding_idx=padding_idx)

    def forward(self, input_ids):
        return self.emb(input_ids)


share_classes(globals())
