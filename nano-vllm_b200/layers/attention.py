"""Paged-KV scatter on a hand-written CUDA kernel, and the attention call.

`store_kvcache` has the signature and preconditions of
nanovllm/layers/attention.py:33-40 (the Triton kernel at :10-30 is replaced by
b2_store_kvcache: 16-byte vector copies, several tokens per CTA, bit-exact).
`Attention` keeps the reference's interface (:43-75).  The attention
arithmetic itself stays a library call, as in the reference: flash-attn's
varlen kernel for prefill and its paged kv-cache kernel for decode.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..utils.context import get_context

try:  # the attention library is outside this path; it is only called, never re-implemented
    from flash_attn import flash_attn_varlen_func, flash_attn_with_kvcache
except Exception:  # pragma: no cover
    flash_attn_varlen_func = flash_attn_with_kvcache = None


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor):
    ops.store_kvcache(key, value, k_cache, v_cache, slot_mapping)


def _sdpa_paged(q, k_cache, v_cache, context_lens, block_tables, scale, q_lens=None):
    """Plain-PyTorch attention over the paged cache: a slow stand-in for the
    library call, used for small shapes when flash-attn cannot run."""
    nh, hd = q.shape[-2], q.shape[-1]
    nkv = k_cache.shape[-2]
    bs = k_cache.shape[1]
    outs = []
    off = 0
    lens = context_lens.tolist()
    for i, n_ctx in enumerate(lens):
        tq = 1 if q_lens is None else q_lens[i]
        if n_ctx == 0:
            outs.append(torch.zeros(tq, nh, hd, dtype=q.dtype, device=q.device))
            off += tq
            continue
        nblk = (n_ctx + bs - 1) // bs
        blocks = block_tables[i, :nblk].long()
        k = k_cache[blocks].reshape(-1, nkv, hd)[:n_ctx]
        v = v_cache[blocks].reshape(-1, nkv, hd)[:n_ctx]
        qi = q[off:off + tq]
        mask = None
        if tq > 1:
            qpos = torch.arange(tq, device=q.device).unsqueeze(1) + (n_ctx - tq)
            mask = torch.arange(n_ctx, device=q.device).unsqueeze(0) <= qpos
        o = torch.nn.functional.scaled_dot_product_attention(qi.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                                             v.transpose(0, 1).unsqueeze(0), attn_mask=mask, scale=scale, enable_gqa=True)
        outs.append(o.squeeze(0).transpose(0, 1))
        off += tq
    return torch.cat(outs)


class Attention(nn.Module):
    # "flash_attn" (the reference's library call) or "sdpa" (plain PyTorch, for tests on small shapes when flash-attn cannot run)
    backend = "flash_attn"

    def __init__(self, num_heads, head_dim, scale, num_kv_heads):
        super().__init__()
        self.num_heads, self.head_dim, self.scale, self.num_kv_heads = num_heads, head_dim, scale, num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Attention over K/V that are already in the paged cache (decode, or
        prefill with a cached prefix) or passed in (plain prefill)."""
        ctx = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if Attention.backend == "sdpa":
            if ctx.is_prefill:
                cu_q, cu_k = ctx.cu_seqlens_q.tolist(), ctx.cu_seqlens_k.tolist()
                q_lens = [b - a for a, b in zip(cu_q[:-1], cu_q[1:])]
                k_lens = torch.tensor([b - a for a, b in zip(cu_k[:-1], cu_k[1:])])
                if ctx.block_tables is None:  # no cache bound (warm-up) or no prefix: attend over the passed K/V
                    outs = []
                    for i, (a, b) in enumerate(zip(cu_q[:-1], cu_q[1:])):
                        o = torch.nn.functional.scaled_dot_product_attention(
                            q[a:b].transpose(0, 1).unsqueeze(0), k[a:b].transpose(0, 1).unsqueeze(0), v[a:b].transpose(0, 1).unsqueeze(0),
                            is_causal=True, scale=self.scale, enable_gqa=True)
                        outs.append(o.squeeze(0).transpose(0, 1))
                    return torch.cat(outs)
                return _sdpa_paged(q, k_cache, v_cache, k_lens, ctx.block_tables, self.scale, q_lens)
            return _sdpa_paged(q, k_cache, v_cache, ctx.context_lens, ctx.block_tables, self.scale)
        if flash_attn_varlen_func is None:
            raise RuntimeError("flash-attn is not importable; set Attention.backend = 'sdpa' for small test shapes")
        if ctx.is_prefill:
            if ctx.block_tables is not None:  # prefix cache / chunked prefill: read K/V from the cache
                k, v = k_cache, v_cache
            return flash_attn_varlen_func(q, k, v, max_seqlen_q=ctx.max_seqlen_q, cu_seqlens_q=ctx.cu_seqlens_q,
                                          max_seqlen_k=ctx.max_seqlen_k, cu_seqlens_k=ctx.cu_seqlens_k,
                                          softmax_scale=self.scale, causal=True, block_table=ctx.block_tables)
        return flash_attn_with_kvcache(q.unsqueeze(1), k_cache, v_cache, cache_seqlens=ctx.context_lens,
                                       block_table=ctx.block_tables, softmax_scale=self.scale, causal=True).squeeze(1)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """Reference behaviour: scatter this step's K/V into the cache (when one is bound), then attend."""
        if self.k_cache.numel() and self.v_cache.numel():
            store_kvcache(k, v, self.k_cache, self.v_cache, get_context().slot_mapping)
        return self.attend(q, k, v)
