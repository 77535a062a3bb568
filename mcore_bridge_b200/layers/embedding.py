"""Vocab-parallel token embedding (rows sharded over TP; out-of-shard ids contribute zero, then reduce)."""
from __future__ import annotations

import torch
from torch import nn

from ..parallel import mappings as M
from ..parallel import state as ps
from .linear import _set_tp_attrs


class VocabParallelEmbedding(nn.Module):

    def __init__(self, num_embeddings: int, embedding_dim: int, config):
        super().__init__()
        self.config = config
        n = ps.get_world_size('tp')
        assert num_embeddings % n == 0, 'vocab must be padded to a multiple of TP'
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.per_partition = num_embeddings // n
        self.vocab_start = ps.get_rank_in('tp') * self.per_partition if n > 1 else 0
        self.tp = n
        self.weight = nn.Parameter(torch.empty(self.per_partition, embedding_dim, dtype=config.params_dtype))
        _set_tp_attrs(self.weight, n > 1, 0)

    def forward(self, input_ids: torch.Tensor, scatter_to_sequence_parallel: bool = False) -> torch.Tensor:
        """``input_ids [T]`` -> ``[T, H]`` (or ``[T/tp, H]`` reduce-scattered for sequence parallelism)."""
        if self.tp > 1:
            local = input_ids - self.vocab_start
            mask = (local < 0) | (local >= self.per_partition)
            out = torch.nn.functional.embedding(local.masked_fill(mask, 0), self.weight)
            out = out.masked_fill(mask[..., None], 0.0)
            if scatter_to_sequence_parallel:
                return M.reduce_scatter_to_sequence_parallel_region(out)
            return M.reduce_from_tensor_model_parallel_region(out)
        return torch.nn.functional.embedding(input_ids, self.weight)


class LanguageModelEmbedding(nn.Module):
    """``embedding.word_embeddings`` wrapper so parameter names match the bridge's expectations."""

    def __init__(self, config, vocab_size: int):
        super().__init__()
        self.config = config
        self.word_embeddings = VocabParallelEmbedding(vocab_size, config.hidden_size, config)

    def forward(self, input_ids, scatter_to_sequence_parallel: bool = False):
        return self.word_embeddings(input_ids, scatter_to_sequence_parallel)
