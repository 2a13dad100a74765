"""Vocabulary-parallel embedding and LM head without NCCL.

Interfaces follow nanovllm/layers/embed_head.py (VocabParallelEmbedding :9-42,
ParallelLMHead :45-66).  The embedding's "masked lookup + all_reduce" becomes
one kernel in which the rank that owns a token id writes its row into every
rank's buffer.  The LM head's "F.linear + gather + cat" becomes a GEMM whose
epilogue stores each rank's slice directly into rank 0's [B, vocab] buffer.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils.context import get_context
from .linear import _tp_rank_world


class VocabParallelEmbedding(nn.Module):

    def __init__(self, num_embeddings: int, embedding_dim: int):
        super().__init__()
        self.tp_rank, self.tp_size = _tp_rank_world()
        assert num_embeddings % self.tp_size == 0
        self.num_embeddings = num_embeddings
        self.num_embeddings_per_partition = num_embeddings // self.tp_size
        self.vocab_start_idx = self.num_embeddings_per_partition * self.tp_rank
        self.vocab_end_idx = self.vocab_start_idx + self.num_embeddings_per_partition
        self.weight = nn.Parameter(torch.empty(self.num_embeddings_per_partition, embedding_dim), requires_grad=False)
        self.weight.weight_loader = self.weight_loader

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        rows = param.data.size(0)
        param.data.copy_(loaded_weight.narrow(0, self.tp_rank * rows, rows))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.embed(x, self.weight, self.vocab_start_idx, self.vocab_end_idx, self.tp_size)


class ParallelLMHead(VocabParallelEmbedding):

    def __init__(self, num_embeddings: int, embedding_dim: int, bias: bool = False):
        assert not bias
        super().__init__(num_embeddings, embedding_dim)

    def forward(self, x: torch.Tensor):
        ctx = get_context()
        return ops.lm_head(x, self.weight, ctx.last_token_index if ctx.is_prefill else None)

    def forward_sample(self, x: torch.Tensor, temperatures: torch.Tensor | None, seed: int, out: torch.Tensor | None = None):
        """forward() followed by Sampler.forward (nanovllm/layers/sampler.py:7-12; greedy when temperatures is
        None) without materialising the logits: every rank scans its vocabulary slice in the GEMM epilogue and
        only the best (score, id) per row reaches rank 0.  Returns int64 token ids, valid on rank 0."""
        ctx = get_context()
        return ops.lm_head_sample(x, self.weight, ctx.last_token_index if ctx.is_prefill else None, temperatures, seed, out)
