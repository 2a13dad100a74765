"""Tensor-level wrappers over the C ABI: they check dtypes and layouts, pick
the current CUDA stream, allocate outputs with torch and pass raw pointers."""
from __future__ import annotations

import ctypes as C

import torch

from . import _abi
from .runtime import get_runtime

_lib = _abi.lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _bf16_rows(t: torch.Tensor, what: str) -> torch.Tensor:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise TypeError(f"{what}: expected a CUDA bf16 tensor, got {t.dtype} on {t.device}")
    if t.stride(-1) != 1:
        t = t.contiguous()
    return t


def _as2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 2:
        return t
    return t.reshape(-1, t.shape[-1])


def gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x[..., K] @ w[N, K]^T (+ bias)."""
    lead = x.shape[:-1]
    x2 = _as2d(_bf16_rows(x, "gemm input"))
    if x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    w = _bf16_rows(w, "gemm weight")
    M, K = x2.shape
    N = w.shape[0]
    if w.dim() != 2 or w.shape[1] != K:
        raise ValueError(f"gemm: input has {K} features, weight is {tuple(w.shape)}")
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if M:
        _abi.check(_lib.b2_gemm(get_runtime().ctx, x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0),
                                bias.data_ptr() if bias is not None else None, out.data_ptr(), out.stride(0), M, N, K, _stream()), "b2_gemm")
    return out.view(*lead, N)


def qkv_fused(x: torch.Tensor, w: torch.Tensor, bias, nq: int, nkv: int, head_dim: int, q_norm_w, k_norm_w, eps: float,
              positions: torch.Tensor, cos_sin: torch.Tensor, k_cache, v_cache, slot_mapping) -> torch.Tensor:
    """qkv projection + q/k head norm + RoPE + KV scatter; returns the [M, (nq + 2 nkv) head_dim] tensor with q and k
    already normalised and rotated."""
    x2 = _as2d(_bf16_rows(x, "qkv input"))
    if x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    M, K = x2.shape
    N = w.shape[0]
    assert N == (nq + 2 * nkv) * head_dim and w.shape[1] == K
    assert positions.dtype == torch.int64 and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    have_cache = k_cache is not None and k_cache.numel() > 0
    if have_cache:
        assert k_cache.stride(1) == nkv * head_dim and slot_mapping.dtype == torch.int32
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if M:
        _abi.check(_lib.b2_qkv_fused(get_runtime().ctx, x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0),
                                     bias.data_ptr() if bias is not None else None, out.data_ptr(), out.stride(0), M, nq, nkv, head_dim, K,
                                     q_norm_w.data_ptr() if q_norm_w is not None else None, k_norm_w.data_ptr() if k_norm_w is not None else None,
                                     float(eps), positions.data_ptr(), cos_sin.data_ptr(), k_cache.data_ptr() if have_cache else None,
                                     v_cache.data_ptr() if have_cache else None, slot_mapping.data_ptr() if have_cache else None, _stream()),
                   "b2_qkv_fused")
    return out


def gemm_silu_mul(x: torch.Tensor, w_pairs: torch.Tensor) -> torch.Tensor:
    """silu(x @ gate^T) * (x @ up^T) where w_pairs interleaves gate and up rows (gate_0, up_0, gate_1, ...)."""
    lead = x.shape[:-1]
    x2 = _as2d(_bf16_rows(x, "gemm_silu_mul input"))
    if x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    M, K = x2.shape
    I = w_pairs.shape[0] // 2
    if w_pairs.shape[1] != K or w_pairs.shape[0] % 2:
        raise ValueError(f"gemm_silu_mul: input has {K} features, paired weight is {tuple(w_pairs.shape)}")
    out = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    if M:
        _abi.check(_lib.b2_gemm_silu_mul(get_runtime().ctx, x2.data_ptr(), x2.stride(0), w_pairs.data_ptr(), w_pairs.stride(0),
                                         out.data_ptr(), out.stride(0), M, I, K, _stream()), "b2_gemm_silu_mul")
    return out.view(*lead, I)


def rowpar_form(M: int, N: int) -> int:
    """Which form of the fused row-parallel block serves M tokens of N features on this runtime
    (_abi.FORM_ONESHOT / FORM_OWNER: b2_rowpar_fused; FORM_TWOSHOT: b2_rowpar_fused_twoshot).  The library decides."""
    form = _lib.b2_rowpar_form(get_runtime().ctx, M, N)
    if form < 0:
        raise _abi.B2Error(f"b2_rowpar_form({M}, {N}): bad argument")
    return form


def rowpar_fused(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor | None,
                 norm_w: torch.Tensor | None, eps: float):
    """Row-parallel GEMM + all-reduce (+ residual add + RMSNorm when norm_w is given).
    Returns y, or (normed, new_residual).

    For many tokens at tensor-parallel size >= 2 (rowpar_form(M, N) == FORM_TWOSHOT) the two-shot kernel runs:
    `normed` is then a view of a buffer owned by the runtime (valid until the next such call) and `new_residual`
    holds only the rows this rank owns (16-row blocks rank, rank + world, ...); the next fused call reads exactly
    those rows."""
    x2 = _as2d(_bf16_rows(x, "row-parallel input"))
    if x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    M, Kr = x2.shape
    N = w.shape[0]
    rt = get_runtime()
    res_out = None
    if norm_w is not None:
        residual = _bf16_rows(residual, "residual")
        if not residual.is_contiguous():
            residual = residual.contiguous()
        res_out = torch.empty_like(residual)
    args_tail = (residual.data_ptr() if norm_w is not None else None, norm_w.data_ptr() if norm_w is not None else None, float(eps))
    if M and rowpar_form(M, N) == _abi.FORM_TWOSHOT:
        ptr = C.c_void_p()
        _abi.check(_lib.b2_rowpar_fused_twoshot(rt.ctx, x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0),
                                                bias.data_ptr() if bias is not None else None, M, N, Kr, *args_tail, C.byref(ptr),
                                                res_out.data_ptr() if res_out is not None else None, _stream()), "b2_rowpar_fused_twoshot")
        out = _library_view(ptr.value, (M, N), x.device)
        if norm_w is None:
            return out.clone().view(*x.shape[:-1], N)  # a plain forward hands out memory the caller may keep
        return out, res_out
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if M:
        _abi.check(_lib.b2_rowpar_fused(rt.ctx, x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0),
                                        bias.data_ptr() if bias is not None else None, M, N, Kr, *args_tail, out.data_ptr(),
                                        res_out.data_ptr() if res_out is not None else None, _stream()), "b2_rowpar_fused")
    if norm_w is None:
        return out.view(*x.shape[:-1], N)
    return out, res_out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = _bf16_rows(x, "rmsnorm input")
    dim = x.shape[-1]
    # rows with a common stride: [rows, dim] views (e.g. q heads inside the qkv output) are taken as they are
    if x.dim() == 2:
        x2 = x
    elif x.is_contiguous():
        x2 = x.view(-1, dim)
    else:
        x2 = x.contiguous().view(-1, dim)
    if x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape, dtype=torch.bfloat16, device=x.device)
    _abi.check(_lib.b2_rmsnorm(x2.data_ptr(), x2.stride(0), w.data_ptr(), float(eps), x2.shape[0], dim, out.data_ptr(), dim, _stream()), "b2_rmsnorm")
    return out.view(x.shape)


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float):
    x = _bf16_rows(x, "add_rmsnorm input").contiguous()
    residual = _bf16_rows(residual, "residual").contiguous()
    dim = x.shape[-1]
    rows = x.numel() // dim
    out, res_out = torch.empty_like(x), torch.empty_like(x)
    _abi.check(_lib.b2_add_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), float(eps), rows, dim, out.data_ptr(), res_out.data_ptr(), _stream()), "b2_add_rmsnorm")
    return out, res_out


def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    n, heads, hd = key.shape
    D = heads * hd
    # the reference's own preconditions (nanovllm/layers/attention.py:36-39)
    assert key.stride(-1) == 1 and value.stride(-1) == 1
    assert key.stride(1) == hd and value.stride(1) == hd
    assert k_cache.stride(1) == D and v_cache.stride(1) == D
    assert slot_mapping.numel() == n
    assert key.element_size() == 2 and k_cache.element_size() == 2 and slot_mapping.dtype == torch.int32
    _abi.check(_lib.b2_store_kvcache(key.data_ptr(), key.stride(0), value.data_ptr(), value.stride(0), k_cache.data_ptr(),
                                     v_cache.data_ptr(), slot_mapping.data_ptr(), n, D, _stream()), "b2_store_kvcache")


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    x2 = _as2d(_bf16_rows(x, "silu_and_mul input"))
    M, two_i = x2.shape
    I = two_i // 2
    out = torch.empty(M, I, dtype=torch.bfloat16, device=x.device)
    _abi.check(_lib.b2_silu_and_mul(x2.data_ptr(), x2.stride(0), M, I, out.data_ptr(), _stream()), "b2_silu_and_mul")
    return out.view(*x.shape[:-1], I)


def qk_norm_rope_store(qkv: torch.Tensor, nq: int, nkv: int, head_dim: int, q_norm_w, k_norm_w, eps: float,
                       positions: torch.Tensor, cos_sin: torch.Tensor, k_cache, v_cache, slot_mapping) -> None:
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.dtype == torch.bfloat16
    assert positions.dtype == torch.int64 and cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
    have_cache = k_cache is not None and k_cache.numel() > 0
    if have_cache:
        assert k_cache.stride(1) == nkv * head_dim and slot_mapping.dtype == torch.int32
    _abi.check(_lib.b2_qk_norm_rope_store(qkv.data_ptr(), qkv.stride(0), qkv.shape[0], nq, nkv, head_dim,
                                          q_norm_w.data_ptr() if q_norm_w is not None else None,
                                          k_norm_w.data_ptr() if k_norm_w is not None else None, float(eps),
                                          positions.data_ptr(), cos_sin.data_ptr(),
                                          k_cache.data_ptr() if have_cache else None, v_cache.data_ptr() if have_cache else None,
                                          slot_mapping.data_ptr() if have_cache else None, _stream()), "b2_qk_norm_rope_store")


def embed(ids: torch.Tensor, w: torch.Tensor, vocab_start: int, vocab_end: int, world: int) -> torch.Tensor:
    assert ids.dtype == torch.int64 and ids.is_cuda
    ids = ids.contiguous()
    M, H = ids.numel(), w.shape[1]
    out = torch.empty(M, H, dtype=w.dtype, device=w.device)
    ctx = get_runtime().ctx if world > 1 else None
    _abi.check(_lib.b2_embed(ctx, ids.data_ptr(), w.data_ptr(), vocab_start, vocab_end, M, H, out.data_ptr(), _stream()), "b2_embed")
    return out.view(*ids.shape, H)


class _DevicePtr:
    """Minimal __cuda_array_interface__ carrier so torch can view library-owned memory."""

    def __init__(self, ptr: int, shape: tuple[int, ...]):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "<u2", "data": (ptr, False), "version": 3, "strides": None}


_LOGIT_VIEWS: dict = {}


def _library_view(ptr: int, shape: tuple[int, int], device) -> torch.Tensor:
    """bf16 tensor over memory the library owns; built once per (address, shape), outside any graph capture."""
    key = (ptr, *shape)
    view = _LOGIT_VIEWS.get(key)
    if view is None:
        view = torch.as_tensor(_DevicePtr(ptr, shape), device=device).view(torch.bfloat16)
        _LOGIT_VIEWS[key] = view
    return view


def lm_head(h: torch.Tensor, w: torch.Tensor, row_index: torch.Tensor | None):
    """Returns the gathered [B, vocab] logits on rank 0 (a view of the runtime's
    buffer, valid until the next call) and None elsewhere."""
    rt = get_runtime()
    h2 = _as2d(_bf16_rows(h, "lm_head input"))
    if h2.stride(0) % 8 != 0 or h2.data_ptr() % 16 != 0:
        h2 = h2.contiguous()
    B = h2.shape[0] if row_index is None else row_index.numel()
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_cuda
    Vr, H = w.shape
    out = C.c_void_p()
    _abi.check(_lib.b2_lm_head(rt.ctx, h2.data_ptr(), h2.stride(0), row_index.data_ptr() if row_index is not None else None,
                               w.data_ptr(), w.stride(0), B, Vr, H, C.byref(out), _stream()), "b2_lm_head")
    if rt.rank != 0:
        return None
    vocab = Vr * rt.world
    key = (out.value, B, vocab)
    view = _LOGIT_VIEWS.get(key)
    if view is None:  # built once per shape (outside any graph capture: the first call of a shape is a warm-up)
        view = torch.as_tensor(_DevicePtr(out.value, (B, vocab)), device=h.device).view(torch.bfloat16)
        _LOGIT_VIEWS[key] = view
    return view


def lm_head_sample(h: torch.Tensor, w: torch.Tensor, row_index: torch.Tensor | None, temperatures: torch.Tensor | None,
                   seed: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """LM head and sampler in one pass over the vocabulary shard (no logits in memory).  Returns int64 token ids
    [B], valid on rank 0 only.  temperatures: fp32 [B] on the device, or None for greedy decoding."""
    rt = get_runtime()
    h2 = _as2d(_bf16_rows(h, "lm_head input"))
    if h2.stride(0) % 8 != 0 or h2.data_ptr() % 16 != 0:
        h2 = h2.contiguous()
    B = h2.shape[0] if row_index is None else row_index.numel()
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_cuda
    if temperatures is not None:
        assert temperatures.dtype == torch.float32 and temperatures.is_cuda and temperatures.is_contiguous() and temperatures.numel() >= B
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=h.device)
    assert out.dtype == torch.int64 and out.is_cuda and out.numel() >= B
    Vr, H = w.shape
    _abi.check(_lib.b2_lm_head_sample(rt.ctx, h2.data_ptr(), h2.stride(0), row_index.data_ptr() if row_index is not None else None,
                                      w.data_ptr(), w.stride(0), B, Vr, H, temperatures.data_ptr() if temperatures is not None else None,
                                      int(seed) & 0xFFFFFFFFFFFFFFFF, out.data_ptr(), _stream()), "b2_lm_head_sample")
    return out[:B]


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    assert logits.dim() == 2 and logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int64, device=logits.device)
    assert out.dtype == torch.int64 and out.numel() >= logits.shape[0]
    _abi.check(_lib.b2_argmax(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1], out.data_ptr(), _stream()), "b2_argmax")
    return out


def broadcast_tokens(buf: torch.Tensor) -> torch.Tensor:
    """Rank 0's int64 token ids into `buf` on every rank (in place)."""
    assert buf.dtype == torch.int64 and buf.is_cuda and buf.is_contiguous()
    _abi.check(_lib.b2_broadcast_tokens(get_runtime().ctx, buf.data_ptr(), buf.numel(), _stream()), "b2_broadcast_tokens")
    return buf


def advance_decode(tokens, input_ids, positions, context_lens, slot_mapping, block_tables, block_size: int, num_slots: int) -> None:
    """Device-side equivalent of building the next decode step's inputs.  num_slots = slots of the KV cache
    (blocks * block_size): a row whose next position has no block, or whose slot would lie outside the cache, is
    frozen (slot -1, position and length unchanged) instead of being sent outside the cache."""
    n = tokens.numel()
    assert tokens.dtype == torch.int64 and positions.dtype == torch.int64 and block_tables.dtype == torch.int32
    assert block_tables.dim() == 2 and block_tables.stride(1) == 1 and block_tables.shape[0] >= n
    _abi.check(_lib.b2_advance_decode(tokens.data_ptr(), input_ids.data_ptr(), positions.data_ptr(), context_lens.data_ptr(),
                                      slot_mapping.data_ptr(), block_tables.data_ptr(), block_tables.stride(0), block_tables.shape[1],
                                      block_size, num_slots, n, _stream()), "b2_advance_decode")
