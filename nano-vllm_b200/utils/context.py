"""Per-step attention metadata shared between the runner and the layers.

Same role and field names as nanovllm/utils/context.py:5-27: the runner fills
it before a forward pass; ParallelLMHead reads `is_prefill` / `cu_seqlens_q`,
the attention layer reads the slot mapping, context lengths and block tables.
"""
from __future__ import annotations

import torch


class Context:
    __slots__ = ("is_prefill", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q", "max_seqlen_k", "slot_mapping",
                 "context_lens", "block_tables", "last_token_index")

    def __init__(self, is_prefill: bool = False, cu_seqlens_q: torch.Tensor | None = None, cu_seqlens_k: torch.Tensor | None = None,
                 max_seqlen_q: int = 0, max_seqlen_k: int = 0, slot_mapping: torch.Tensor | None = None,
                 context_lens: torch.Tensor | None = None, block_tables: torch.Tensor | None = None):
        self.is_prefill = is_prefill
        self.cu_seqlens_q, self.cu_seqlens_k = cu_seqlens_q, cu_seqlens_k
        self.max_seqlen_q, self.max_seqlen_k = max_seqlen_q, max_seqlen_k
        self.slot_mapping, self.context_lens, self.block_tables = slot_mapping, context_lens, block_tables
        # int32 index of the last token of every sequence (cu_seqlens_q[1:] - 1), built once per prefill step
        self.last_token_index = (cu_seqlens_q[1:] - 1).to(torch.int32) if (is_prefill and cu_seqlens_q is not None) else None


_current = Context()


def get_context() -> Context:
    return _current


def set_context(is_prefill, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0, max_seqlen_k=0, slot_mapping=None,
                context_lens=None, block_tables=None) -> None:
    global _current
    _current = Context(is_prefill, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, slot_mapping, context_lens, block_tables)


def reset_context() -> None:
    global _current
    _current = Context()
