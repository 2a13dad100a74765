"""Rotary position table (nanovllm/layers/rotary_embedding.py:17-59).

Only the cos||sin table lives here; the rotation itself runs inside the fused
q/k-norm + RoPE + KV-scatter kernel (ops.qk_norm_rope_store).
"""
from __future__ import annotations

from functools import lru_cache

import torch
from torch import nn


class RotaryEmbedding(nn.Module):

    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float) -> None:
        super().__init__()
        assert rotary_dim == head_size
        self.head_size = head_size
        exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float, device="cpu") / rotary_dim
        inv_freq = 1.0 / (base ** exponents)
        angles = torch.outer(torch.arange(max_position_embeddings, dtype=torch.float, device="cpu"), inv_freq)
        table = torch.cat((angles.cos(), angles.sin()), dim=-1)  # [max_pos, head_size], fp32
        self.register_buffer("cos_sin_cache", table.to(torch.get_default_device() if hasattr(torch, "get_default_device") else "cpu"), persistent=False)


@lru_cache(1)
def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float) -> RotaryEmbedding:
    return RotaryEmbedding(head_size, rotary_dim, max_position, base)
