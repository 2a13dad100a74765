"""CPU oracle for the tensor-parallel transformer-layer path of nano-vllm.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain PyTorch on the CPU,
the arithmetic of the reference's tensor-parallel layer path so that the CUDA
library can be checked against it.  Nothing on the product path may import it:
only tests, the smoke check and the CPU-baseline leg of the benchmark do.

Parity pin: the reference ships no tests or golden vectors for this path.  The
restatement is pinned instead against outputs of the reference's own modules
(imported from its source tree under a 2-rank gloo group) stored as fixtures
under tests/golden/ by tests/golden/make_golden.py.

Every function names the reference lines it follows (paths are relative to the
reference project root).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

# --------------------------------------------------------------------------
# sharding helpers (weight loaders)
# --------------------------------------------------------------------------


def shard_column(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Output-dimension shard of a [out, in] weight.

    nanovllm/layers/linear.py:65-70 (ColumnParallelLinear.weight_loader):
    narrow dim 0 to rows [rank*out/world, (rank+1)*out/world).
    """
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].clone()


def shard_row(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Input-dimension shard of a [out, in] weight.

    nanovllm/layers/linear.py:142-150 (RowParallelLinear.weight_loader):
    narrow dim 1 to columns [rank*in/world, (rank+1)*in/world).
    """
    k = w.shape[1] // world
    return w[:, rank * k:(rank + 1) * k].clone()


def shard_merged(ws: list[torch.Tensor], rank: int, world: int) -> torch.Tensor:
    """Rank-local weight of a merged column-parallel layer (gate_up_proj).

    nanovllm/layers/linear.py:87-93: shard `i` of size out_i is chunked over
    ranks and placed at row offset sum(out[:i])/world.
    """
    return torch.cat([w.chunk(world, 0)[rank] for w in ws], 0).clone()


def shard_qkv(wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank-local qkv weight: [q heads of rank; k heads of rank; v heads of rank].

    nanovllm/layers/linear.py:114-128.
    """
    return torch.cat([wq.chunk(world, 0)[rank], wk.chunk(world, 0)[rank], wv.chunk(world, 0)[rank]], 0).clone()


# --------------------------------------------------------------------------
# linear layers
# --------------------------------------------------------------------------


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ w.T (+ bias): fp32 accumulation, one rounding to the input dtype.

    nanovllm/layers/linear.py:51,73 (F.linear).  cuBLAS accumulates bf16
    products in fp32 and rounds once, which is what this does.
    """
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def row_parallel_partials(xs: list[torch.Tensor], ws: list[torch.Tensor], bias: torch.Tensor | None = None) -> list[torch.Tensor]:
    """Per-rank partial products of RowParallelLinear, rounded to the I/O dtype.

    nanovllm/layers/linear.py:153: y = F.linear(x, W, bias if rank == 0 else None)
    is materialised in the activation dtype before the collective.
    """
    return [linear(x, w, bias if r == 0 else None) for r, (x, w) in enumerate(zip(xs, ws))]


def all_reduce_sum(parts: list[torch.Tensor]) -> torch.Tensor:
    """Sum over ranks (nanovllm/layers/linear.py:155, dist.all_reduce).

    The order and intermediate precision of NCCL's reduction are not part of
    the reference's contract; the oracle sums the rounded partials in fp32 and
    rounds once, the most accurate result any order can give.
    """
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        acc += p.float()
    return acc.to(parts[0].dtype)


def row_parallel_linear(xs, ws, bias=None) -> torch.Tensor:
    """RowParallelLinear.forward over all ranks (nanovllm/layers/linear.py:152-156)."""
    parts = row_parallel_partials(xs, ws, bias)
    return all_reduce_sum(parts) if len(parts) > 1 else parts[0]


# --------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """nanovllm/layers/layernorm.py:16-26.

    fp32 statistics; the normalised value is rounded to the I/O dtype and then
    multiplied by the weight in that dtype (a second rounding).
    """
    dt = x.dtype
    x32 = x.float()
    var = x32.pow(2).mean(dim=-1, keepdim=True)
    x32 = x32 * torch.rsqrt(var + eps)
    return x32.to(dt) * weight.to(dt)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """nanovllm/layers/layernorm.py:28-40.  Returns (normed, new_residual).

    s = fp32(x) + fp32(residual); new_residual = round(s); statistics and
    scaling use the un-rounded fp32 s; the result is rounded and then
    multiplied by the weight in the I/O dtype.
    (In fp32 the reference aliases its returned residual with the normed
    output; the value restated here is the intended one, x + residual.)
    """
    dt = x.dtype
    s = x.float() + residual.float()
    new_res = s.to(dt)
    var = s.pow(2).mean(dim=-1, keepdim=True)
    normed = (s * torch.rsqrt(var + eps)).to(dt) * weight.to(dt)
    return normed, new_res


def fused_row_parallel_norm(xs, ws, residual, norm_weight, eps):
    """RowParallelLinear -> all_reduce -> add + RMSNorm, as wired by
    nanovllm/models/qwen3.py:155-157 (o_proj -> post_attention_layernorm) and
    :158 -> next layer :155 (down_proj -> input_layernorm), with the
    reference's roundings: partial -> I/O dtype, sum -> I/O dtype, then
    add_rms_norm."""
    y = row_parallel_linear(xs, ws)
    return add_rms_norm(y, residual, norm_weight, eps)


def fused_row_parallel_norm_exact(xs, ws, residual, norm_weight, eps):
    """The same block with no intermediate rounding (fp32 throughout): the
    'fp32 reference' the bf16 tolerances are stated against."""
    y = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
    s = y + residual.float()
    var = s.pow(2).mean(dim=-1, keepdim=True)
    return s * torch.rsqrt(var + eps) * norm_weight.float(), s


# --------------------------------------------------------------------------
# embedding / LM head
# --------------------------------------------------------------------------


def vocab_parallel_embedding(ids: torch.Tensor, w_shards: list[torch.Tensor]) -> torch.Tensor:
    """nanovllm/layers/embed_head.py:34-42.

    Per rank: mask ids outside [start, end), look up (id - start) * mask, zero
    masked rows; then all_reduce(sum).  Exactly one rank contributes a
    non-zero row, so the sum is exact.
    """
    world = len(w_shards)
    per = w_shards[0].shape[0]
    out = torch.zeros(ids.numel(), w_shards[0].shape[1], dtype=torch.float32)
    for r in range(world):
        start, end = r * per, (r + 1) * per
        mask = (ids >= start) & (ids < end)
        local = mask * (ids - start)
        y = w_shards[r][local].float() * mask.unsqueeze(1)
        out += y
    return out.to(w_shards[0].dtype)


def parallel_lm_head(h: torch.Tensor, w_shards: list[torch.Tensor], last_indices: torch.Tensor | None = None) -> torch.Tensor:
    """nanovllm/layers/embed_head.py:56-66.

    Prefill keeps the last token of every sequence (cu_seqlens_q[1:] - 1);
    each rank multiplies by its vocab shard; rank 0 concatenates the shards
    along the vocab dimension.
    """
    if last_indices is not None:
        h = h[last_indices].contiguous()
    return torch.cat([linear(h, w) for w in w_shards], dim=-1)


# --------------------------------------------------------------------------
# paged KV scatter (integer/byte exact)
# --------------------------------------------------------------------------


# --------------------------------------------------------------------------
# sampler
# --------------------------------------------------------------------------


def sampler_with_noise(logits: torch.Tensor, temperatures: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """nanovllm/layers/sampler.py:9-11 with the exponential noise passed in instead of drawn:
    probs = softmax(float(logits) / T); token = argmax(probs / clamp_min(E, 1e-10))."""
    scaled = logits.float() / temperatures.float().unsqueeze(1)
    probs = torch.softmax(scaled, dim=-1)
    return (probs / noise.float().clamp_min(1e-10)).argmax(dim=-1)


def sampler_scores(logits: torch.Tensor, temperatures: torch.Tensor | None, noise: torch.Tensor | None) -> torch.Tensor:
    """The same draw without the softmax: the denominator of softmax is common to a row and log is monotone, so
    argmax_i p_i / E_i = argmax_i (logit_i / T - log E_i).  Returns the fp64 scores whose row-wise argmax is the
    token; this is the form the fused LM-head sampler evaluates shard by shard.  temperatures None = greedy."""
    z = logits.float().double()
    if temperatures is None:
        return z
    return z / temperatures.double().unsqueeze(1) - torch.log(noise.double().clamp_min(1e-10))


_PHILOX_M0, _PHILOX_M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_PHILOX_W0, _PHILOX_W1 = 0x9E3779B9, 0xBB67AE85
SAMPLE_TAG = 0x53414D50


def philox4x32_10(counter: np.ndarray, key: tuple[int, int]) -> np.ndarray:
    """Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11), vectorised:
    counter uint32 [..., 4] -> uint32 [..., 4].  Each round: (hi0, lo0) = M0 * c0, (hi1, lo1) = M1 * c2,
    c = (hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0), then the key is bumped by the Weyl constants."""
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = _PHILOX_M0 * c[0], _PHILOX_M1 * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0), p1 & mask, (p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1), p0 & mask]
        k0, k1 = (k0 + _PHILOX_W0) & 0xFFFFFFFF, (k1 + _PHILOX_W1) & 0xFFFFFFFF
    return np.stack(c, axis=-1).astype(np.uint32)


def fused_sampler_noise(seed: int, call: int, rows: int, vocab: int) -> torch.Tensor:
    """The Exp(1) noise the fused LM-head sampler uses in call number `call`: [rows, vocab] fp64.
    Counter = (vocab id, row // 4, call, tag), key = seed; word row % 4 of the output; 23 bits -> u in (0, 1)."""
    v = np.arange(vocab, dtype=np.uint32)
    out = np.empty((rows, vocab), dtype=np.float64)
    for grp in range((rows + 3) // 4):
        ctr = np.stack([v, np.full_like(v, grp), np.full_like(v, call & 0xFFFFFFFF), np.full_like(v, SAMPLE_TAG)], axis=-1)
        r = philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF))
        for i in range(4):
            row = grp * 4 + i
            if row < rows:
                u = ((r[:, i] >> np.uint32(9)).astype(np.float64) + 0.5) * 2.0 ** -23
                out[row] = -np.log(u)
    return torch.from_numpy(out)


def store_kvcache(key: np.ndarray, value: np.ndarray, k_cache: np.ndarray, v_cache: np.ndarray, slot_mapping: np.ndarray) -> None:
    """nanovllm/layers/attention.py:10-30,33-40, on raw 16-bit words.

    key/value: [N, D] uint16 views of the token rows (rows may come from a
    strided tensor; pass the materialised rows).  k_cache/v_cache: [slots, D]
    uint16, modified in place.  Token i goes to row slot_mapping[i]; -1 skips.
    """
    n, d = key.shape
    assert value.shape == (n, d) and slot_mapping.shape == (n,)
    assert k_cache.shape[1] == d and v_cache.shape[1] == d
    for i in range(n):
        s = int(slot_mapping[i])
        if s == -1:
            continue
        k_cache[s, :] = key[i]
        v_cache[s, :] = value[i]


def store_kvcache_vectorised(key, value, k_cache, v_cache, slot_mapping) -> None:
    """Same result as store_kvcache when the non-negative slots are distinct
    (they always are: one slot per token), for sizes the loop is too slow for."""
    keep = slot_mapping != -1
    k_cache[slot_mapping[keep]] = key[keep]
    v_cache[slot_mapping[keep]] = value[keep]


# --------------------------------------------------------------------------
# elementwise neighbours of the path
# --------------------------------------------------------------------------


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """nanovllm/layers/activation.py:8-11: silu(x[:, :I]) * x[:, I:].

    Eagerly, F.silu on bf16 computes in fp32 and rounds, then the product is
    rounded again; the compiled form keeps fp32 until one final rounding.  The
    oracle follows the eager source (two roundings); tests allow 1 ulp.
    """
    g, u = x.chunk(2, -1)
    return torch.nn.functional.silu(g.float()).to(x.dtype) * u


def rope_cache(head_dim: int, max_pos: int, base: float) -> torch.Tensor:
    """cos||sin table [max_pos, head_dim], fp32 (nanovllm/layers/rotary_embedding.py:27-34)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
    """Neox-style rotation of [T, heads, head_dim] (nanovllm/layers/rotary_embedding.py:6-14,43-47)."""
    cs = cache[positions].unsqueeze(1)
    cos, sin = cs.chunk(2, dim=-1)
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)


# --------------------------------------------------------------------------
# a whole tensor-parallel Qwen3 forward, all ranks in one process
# --------------------------------------------------------------------------


@dataclass
class QwenShape:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate: int
    n_layers: int
    vocab: int
    eps: float = 1e-6
    rope_theta: float = 1e6
    tie: bool = False


def init_full_weights(shape: QwenShape, seed: int, dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    """Seeded N(0, 0.02) full (unsharded) weights under HF parameter names; norm
    weights ~U(0.5, 1.5) so that a dropped norm weight is visible."""
    g = torch.Generator().manual_seed(seed)

    def nrm(*s):
        return (torch.randn(*s, generator=g) * 0.02).to(dtype)

    def uni(n):
        return (torch.rand(n, generator=g) + 0.5).to(dtype)

    H, hd = shape.hidden, shape.head_dim
    w = {"model.embed_tokens.weight": nrm(shape.vocab, H), "model.norm.weight": uni(H)}
    for i in range(shape.n_layers):
        p = f"model.layers.{i}."
        w[p + "self_attn.q_proj.weight"] = nrm(shape.n_heads * hd, H)
        w[p + "self_attn.k_proj.weight"] = nrm(shape.n_kv_heads * hd, H)
        w[p + "self_attn.v_proj.weight"] = nrm(shape.n_kv_heads * hd, H)
        w[p + "self_attn.o_proj.weight"] = nrm(H, shape.n_heads * hd)
        w[p + "self_attn.q_norm.weight"] = uni(hd)
        w[p + "self_attn.k_norm.weight"] = uni(hd)
        w[p + "mlp.gate_proj.weight"] = nrm(shape.intermediate, H)
        w[p + "mlp.up_proj.weight"] = nrm(shape.intermediate, H)
        w[p + "mlp.down_proj.weight"] = nrm(H, shape.intermediate)
        w[p + "input_layernorm.weight"] = uni(H)
        w[p + "post_attention_layernorm.weight"] = uni(H)
    w["lm_head.weight"] = w["model.embed_tokens.weight"] if shape.tie else nrm(shape.vocab, H)
    return w


def _attention_dense(q, k_ctx, v_ctx, scale):
    """softmax(q k^T * scale) v for one sequence; q [Tq, nh, hd], k/v [Tk, nkv, hd];
    causal with the query block aligned to the END of the keys (what
    flash-attn's causal=True does for Tq < Tk)."""
    tq, nh, hd = q.shape
    tk, nkv, _ = k_ctx.shape
    rep = nh // nkv
    kf = k_ctx.float().repeat_interleave(rep, dim=1)
    vf = v_ctx.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kf) * scale
    qi = torch.arange(tq).unsqueeze(1) + (tk - tq)
    ki = torch.arange(tk).unsqueeze(0)
    s = s.masked_fill((ki > qi).unsqueeze(0), float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, vf).to(q.dtype)


class QwenOracle:
    """All-ranks-in-one-process restatement of Qwen3ForCausalLM under tensor
    parallelism (nanovllm/models/qwen3.py:72-88,113-117,146-159,173-183,212-216),
    with a dense KV history per sequence in place of the paged cache and a
    plain softmax attention in place of flash-attn (a library outside the
    path).  Used for token-parity checks on small random-init models."""

    def __init__(self, shape: QwenShape, weights: dict[str, torch.Tensor], world: int, max_pos: int = 4096):
        self.s, self.w, self.world = shape, weights, world
        self.cache = rope_cache(shape.head_dim, max_pos, shape.rope_theta)
        # kv[layer][seq] -> (k [T, nkv, hd], v [T, nkv, hd]) with all kv heads
        self.kv: list[dict[int, tuple[torch.Tensor, torch.Tensor]]] = [dict() for _ in range(shape.n_layers)]

    def _layer(self, li, h, residual, positions, seq_ids, seq_lens):
        s, w, W = self.s, self.w, self.world
        p = f"model.layers.{li}."
        if residual is None:
            residual, h = h, rms_norm(h, w[p + "input_layernorm.weight"], s.eps)
        else:
            h, residual = add_rms_norm(h, residual, w[p + "input_layernorm.weight"], s.eps)
        hd = s.head_dim
        attn_out_shards = []
        wo = w[p + "self_attn.o_proj.weight"]
        for r in range(W):
            wqkv = shard_qkv(w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"], r, W)
            qkv = linear(h, wqkv)
            nq, nkv = s.n_heads // W, s.n_kv_heads // W
            q, k, v = qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
            q = rms_norm(q.reshape(-1, nq, hd), w[p + "self_attn.q_norm.weight"], s.eps)
            k = rms_norm(k.reshape(-1, nkv, hd), w[p + "self_attn.k_norm.weight"], s.eps)
            v = v.reshape(-1, nkv, hd)
            q = apply_rope(q, positions, self.cache)
            k = apply_rope(k, positions, self.cache)
            outs, off = [], 0
            for sid, n in zip(seq_ids, seq_lens):
                key = (sid, r)
                kk, vv = k[off:off + n], v[off:off + n]
                if key in self.kv[li]:
                    pk, pv = self.kv[li][key]
                    kk, vv = torch.cat([pk, kk]), torch.cat([pv, vv])
                self.kv[li][key] = (kk, vv)
                outs.append(_attention_dense(q[off:off + n], kk, vv, hd ** -0.5))
                off += n
            attn_out_shards.append(torch.cat(outs).flatten(1))
        xs = attn_out_shards
        ws = [shard_row(wo, r, W) for r in range(W)]
        h, residual = fused_row_parallel_norm(xs, ws, residual, w[p + "post_attention_layernorm.weight"], s.eps)
        acts, wds = [], []
        for r in range(W):
            wgu = shard_merged([w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"]], r, W)
            acts.append(silu_and_mul(linear(h, wgu)))
            wds.append(shard_row(w[p + "mlp.down_proj.weight"], r, W))
        return row_parallel_linear(acts, wds), residual

    def forward(self, ids, positions, seq_ids, seq_lens):
        """ids/positions: flat int64 [T]; seq_ids/seq_lens: which sequence each
        run of tokens belongs to (new tokens are appended to its KV history).
        Returns logits [len(seq_ids), vocab] for the last token of each run."""
        s, w, W = self.s, self.w, self.world
        emb = w["model.embed_tokens.weight"]
        h = vocab_parallel_embedding(ids, [shard_column(emb, r, W) for r in range(W)])
        residual = None
        for li in range(s.n_layers):
            h, residual = self._layer(li, h, residual, positions, seq_ids, seq_lens)
        h, _ = add_rms_norm(h, residual, w["model.norm.weight"], s.eps)
        last = torch.tensor(seq_lens).cumsum(0) - 1
        head = w["lm_head.weight"]
        return parallel_lm_head(h, [shard_column(head, r, W) for r in range(W)], last)


# --------------------------------------------------------------------------
# seeded input generators shared by tests, fixtures and the benchmark
# --------------------------------------------------------------------------


def rowpar_case(m: int, k_total: int, n: int, world: int, seed: int, dtype=torch.bfloat16):
    """Inputs of one fused row-parallel block: activations ~N(0,1), weights
    ~N(0,0.02), residual ~N(0,1), norm weight ~U(0.5,1.5)."""
    g = torch.Generator().manual_seed(seed)
    kr = k_total // world
    xs = [torch.randn(m, kr, generator=g).to(dtype) for _ in range(world)]
    ws = [(torch.randn(n, kr, generator=g) * 0.02).to(dtype) for _ in range(world)]
    residual = torch.randn(m, n, generator=g).to(dtype)
    norm_w = (torch.rand(n, generator=g) + 0.5).to(dtype)
    return xs, ws, residual, norm_w


def kv_case(n_tokens: int, d: int, num_slots: int, seed: int, frac_skipped: float = 0.1):
    """Random 16-bit K/V rows, a random injective slot mapping with some -1s."""
    rng = np.random.default_rng(seed)
    key = rng.integers(0, 1 << 16, size=(n_tokens, d), dtype=np.uint16)
    value = rng.integers(0, 1 << 16, size=(n_tokens, d), dtype=np.uint16)
    slots = rng.permutation(num_slots)[:n_tokens].astype(np.int32)
    if n_tokens:
        skip = rng.random(n_tokens) < frac_skipped
        slots[skip] = -1
    return key, value, slots


def rowpar_roofline_us(m: int, n: int, kr: int, world: int, bf16_tflops: float, hbm_gbs: float, nvlink_gbs: float) -> dict:
    """Algorithmic work of one fused row-parallel call on one GPU and the time
    each resource needs for it: flops 2*M*N*Kr; NVLink egress 2*(tp-1)/tp*M*N*2 B;
    HBM 2*(M*Kr + N*Kr + 3*M*N + N) B."""
    flops = 2.0 * m * n * kr
    nvl = 2.0 * (world - 1) / world * m * n * 2
    hbm = 2.0 * (m * kr + n * kr + 3 * m * n + n)
    t = {"flops_us": flops / (bf16_tflops * 1e12) * 1e6, "nvlink_us": nvl / (nvlink_gbs * 1e9) * 1e6, "hbm_us": hbm / (hbm_gbs * 1e9) * 1e6}
    t["roof_us"] = max(t.values())
    t.update(flops=flops, nvlink_bytes=nvl, hbm_bytes=hbm)
    return t
