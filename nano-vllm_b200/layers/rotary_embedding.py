"""Rotary position embedding (nanovllm/layers/rotary_embedding.py:17-59).

The decoder layer does not call `forward`: its rotation runs inside the qkv
projection's epilogue (or the q/k-norm + RoPE + KV-scatter kernel) on the same
cos||sin table.  `forward(positions, query, key)` keeps the reference's class
usable on its own (:37-48): it runs that kernel with the head norm and the
KV scatter switched off.
"""
from __future__ import annotations

from functools import lru_cache

import torch
from torch import nn

from .. import ops


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

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """query [T, heads, head_size], key [T, kv_heads, head_size] (or flattened over the heads); returns rotated
        copies, fp32 arithmetic and one rounding to bf16, as the reference's apply_rotary_emb (:6-14)."""
        hd = self.head_size
        t = positions.numel()
        q2, k2 = query.reshape(t, -1), key.reshape(t, -1)
        nq, nkv = q2.shape[1] // hd, k2.shape[1] // hd
        # the kernel works in place on a [T, (nq + 2 nkv) hd] row (q heads, k heads, v heads): the v part stays unused
        buf = torch.empty(t, (nq + 2 * nkv) * hd, dtype=torch.bfloat16, device=query.device)
        buf[:, :nq * hd] = q2
        buf[:, nq * hd:(nq + nkv) * hd] = k2
        ops.qk_norm_rope_store(buf, nq, nkv, hd, None, None, 0.0, positions.reshape(-1).to(torch.int64), self.cos_sin_cache, None, None, None)
        return buf[:, :nq * hd].reshape(query.shape), buf[:, nq * hd:(nq + nkv) * hd].reshape(key.shape)


@lru_cache(1)
def get_rope(head_size: int, rotary_dim: int, max_position: int, base: float) -> RotaryEmbedding:
    return RotaryEmbedding(head_size, rotary_dim, max_position, base)
