"""HBM-bound kernels against the CPU oracle and the golden fixtures (B200)."""
import os

import numpy as np
import pytest
import torch

from oracle import tp_path as O
from tests.gpu_util import assert_close_bf16, ensure_group, ulp_mismatch_fraction

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops(pkg):
    ensure_group()
    from nanovllm_b200 import ops as _ops
    return _ops


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16)).to(DEV).view(torch.bfloat16)


@pytest.mark.parametrize("n,heads,slots_total,strided_v", [(0, 8, 512, False), (1, 1, 256, False), (37, 2, 1024, True), (64, 8, 2048, True),
                                                           (300, 4, 4096, False), (513, 8, 1024, True)])
def test_store_kvcache_bit_exact(ops, n, heads, slots_total, strided_v):
    d = heads * 128
    key, value, slots = O.kv_case(n, d, slots_total, seed=n + heads, frac_skipped=0.25)
    rng = np.random.default_rng(5)
    kc0 = rng.integers(0, 1 << 16, size=(slots_total, d), dtype=np.uint16)
    vc0 = rng.integers(0, 1 << 16, size=(slots_total, d), dtype=np.uint16)
    kc, vc = kc0.copy(), vc0.copy()
    O.store_kvcache(key, value, kc, vc, slots)
    tk = _from_bits(key).view(n, heads, 128)
    if strided_v:  # V as a view into a wider row, like the slice of the qkv GEMM output
        wide = torch.zeros(n, 3 * d, dtype=torch.bfloat16, device=DEV)
        wide[:, 2 * d:] = _from_bits(value)
        tv = wide[:, 2 * d:].view(n, heads, 128)
        assert tv.stride(0) == 3 * d
    else:
        tv = _from_bits(value).view(n, heads, 128)
    gk = _from_bits(kc0).view(slots_total // 256, 256, heads, 128).clone()
    gv = _from_bits(vc0).view(slots_total // 256, 256, heads, 128).clone()
    ops.store_kvcache(tk, tv, gk, gv, torch.from_numpy(slots).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(gk).reshape(slots_total, d), kc)
    assert np.array_equal(_bits(gv).reshape(slots_total, d), vc)


@pytest.mark.parametrize("d", [128, 1024])
def test_store_kvcache_long_prefill_shape(ops, d):
    """16384 tokens per step, slots from a random permutation of 256-token
    blocks (the long-context prefill configuration), checked by the
    vectorised oracle and by a checksum of the untouched slots."""
    n, block, nblocks = 16384, 256, 160
    rng = np.random.default_rng(9)
    key = rng.integers(0, 1 << 16, size=(n, d), dtype=np.uint16)
    value = rng.integers(0, 1 << 16, size=(n, d), dtype=np.uint16)
    perm = rng.permutation(nblocks)
    slots = (perm[np.arange(n) // block] * block + np.arange(n) % block).astype(np.int32)
    kc = np.zeros((nblocks * block, d), np.uint16)
    vc = np.zeros((nblocks * block, d), np.uint16)
    O.store_kvcache_vectorised(key, value, kc, vc, slots)
    gk = torch.zeros(nblocks, block, d // 128, 128, dtype=torch.bfloat16, device=DEV)
    gv = torch.zeros_like(gk)
    ops.store_kvcache(_from_bits(key).view(n, d // 128, 128), _from_bits(value).view(n, d // 128, 128), gk, gv, torch.from_numpy(slots).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(gk).reshape(-1, d), kc)
    assert np.array_equal(_bits(gv).reshape(-1, d), vc)
    # idempotence: scattering the same rows again changes nothing
    ops.store_kvcache(_from_bits(key).view(n, d // 128, 128), _from_bits(value).view(n, d // 128, 128), gk, gv, torch.from_numpy(slots).to(DEV))
    torch.cuda.synchronize()
    assert np.array_equal(_bits(gk).reshape(-1, d), kc)


@pytest.mark.parametrize("rows,dim", [(1, 128), (7, 1024), (64, 4096), (33, 5120), (300, 128), (5, 8192)])
def test_rmsnorm_and_add_rmsnorm(ops, rows, dim):
    g = torch.Generator().manual_seed(rows * 7 + dim)
    x = torch.randn(rows, dim, generator=g).bfloat16()
    r = torch.randn(rows, dim, generator=g).bfloat16()
    w = (torch.rand(dim, generator=g) + 0.5).bfloat16()
    ref = O.rms_norm(x, w, 1e-6)
    got = ops.rmsnorm(x.to(DEV), w.to(DEV), 1e-6)
    assert ulp_mismatch_fraction(got, ref, 1) == 0.0
    assert ulp_mismatch_fraction(got, ref, 0) < 0.02
    refn, refr = O.add_rms_norm(x, r, w, 1e-6)
    gotn, gotr = ops.add_rmsnorm(x.to(DEV), r.to(DEV), w.to(DEV), 1e-6)
    assert torch.equal(gotr.cpu(), refr)  # the residual sum has one rounding: exact
    assert ulp_mismatch_fraction(gotn, refn, 1) == 0.0
    assert ulp_mismatch_fraction(gotn, refn, 0) < 0.02


def test_rmsnorm_golden(ops, golden_dir):
    d = torch.load(os.path.join(golden_dir, "rp_b.pt"))
    gotn, gotr = ops.add_rmsnorm(d["y"].to(DEV), d["residual"].to(DEV), d["norm_w"].to(DEV), 1e-6)
    assert torch.equal(gotr.cpu(), d["new_res"])
    assert ulp_mismatch_fraction(gotn, d["normed"], 1) == 0.0
    assert ulp_mismatch_fraction(ops.rmsnorm(d["y"].to(DEV), d["norm_w"].to(DEV), 1e-6), d["plain_norm"], 1) == 0.0
    r = torch.load(os.path.join(golden_dir, "rope.pt"))
    # head-dim norm over a [tokens, heads, 64] tensor
    assert ulp_mismatch_fraction(ops.rmsnorm(r["q"].to(DEV), r["norm_w"].to(DEV), 1e-6), r["q_normed"], 1) == 0.0


def test_silu_and_mul(ops, golden_dir):
    d = torch.load(os.path.join(golden_dir, "col.pt"))
    for r in range(2):
        got = ops.silu_and_mul(d[f"gu_y{r}"].to(DEV))
        assert ulp_mismatch_fraction(got, d[f"act{r}"], 1) == 0.0
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(64, 2 * 3072, generator=g) * 3).bfloat16()
    assert ulp_mismatch_fraction(ops.silu_and_mul(x.to(DEV)), O.silu_and_mul(x), 1) == 0.0


@pytest.mark.parametrize("hd,nq,nkv,m", [(128, 4, 2, 9), (128, 32, 8, 64), (64, 4, 2, 11)])
def test_qk_norm_rope_store(ops, hd, nq, nkv, m):
    g = torch.Generator().manual_seed(hd + m)
    max_pos, nblocks = 512, 4
    qkv = torch.randn(m, (nq + 2 * nkv) * hd, generator=g).bfloat16()
    qw = (torch.rand(hd, generator=g) + 0.5).bfloat16()
    kw = (torch.rand(hd, generator=g) + 0.5).bfloat16()
    pos = torch.randint(0, max_pos, (m,), generator=g)
    cache = O.rope_cache(hd, max_pos, 1e6)
    slots = torch.randperm(nblocks * 256, generator=g)[:m].to(torch.int32)
    slots[::5] = -1
    q, k, v = qkv.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    q_ref = O.apply_rope(O.rms_norm(q.reshape(m, nq, hd), qw, 1e-6), pos, cache)
    k_ref = O.apply_rope(O.rms_norm(k.reshape(m, nkv, hd), kw, 1e-6), pos, cache)
    kc = torch.zeros(nblocks, 256, nkv, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    dq = qkv.to(DEV).clone()
    ops.qk_norm_rope_store(dq, nq, nkv, hd, qw.to(DEV), kw.to(DEV), 1e-6, pos.to(DEV), cache.to(DEV), kc, vc, slots.to(DEV))
    torch.cuda.synchronize()
    gq, gk, gv = dq.cpu().split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    assert ulp_mismatch_fraction(gq.reshape(m, nq, hd), q_ref, 1) < 1e-3
    assert ulp_mismatch_fraction(gk.reshape(m, nkv, hd), k_ref, 1) < 1e-3
    assert torch.equal(gv, v)  # V is not modified
    keep = slots >= 0
    kflat, vflat = kc.view(-1, nkv * hd).cpu(), vc.view(-1, nkv * hd).cpu()
    assert torch.equal(kflat[slots[keep].long()], gk[keep])       # the cache holds exactly the rotated K rows
    assert torch.equal(vflat[slots[keep].long()], v[keep])        # and the raw V rows
    untouched = torch.ones(nblocks * 256, dtype=torch.bool)
    untouched[slots[keep].long()] = False
    assert kflat[untouched].abs().sum() == 0 and vflat[untouched].abs().sum() == 0


def test_rope_golden(ops, golden_dir):
    """The reference's RotaryEmbedding outputs (head_dim 64) reproduced by the fused kernel without norm weights."""
    r = torch.load(os.path.join(golden_dir, "rope.pt"))
    m = r["q"].shape[0]
    qkv = torch.cat([r["q"].reshape(m, -1), r["k"].reshape(m, -1), r["k"].reshape(m, -1)], dim=-1).to(DEV).contiguous()
    ops.qk_norm_rope_store(qkv, 4, 2, 64, None, None, 1e-6, r["pos"].to(DEV), r["cache"].to(DEV).contiguous(), None, None, None)
    torch.cuda.synchronize()
    assert torch.equal(qkv[:, :256].cpu().view(m, 4, 64), r["q_out"])
    assert torch.equal(qkv[:, 256:384].cpu().view(m, 2, 64), r["k_out"])


def test_rotary_embedding_class_forward_golden(pkg, golden_dir):
    """RotaryEmbedding.forward(positions, query, key), the reference's class surface
    (nanovllm/layers/rotary_embedding.py:37-48), against the reference's own outputs."""
    from nanovllm_b200.layers.rotary_embedding import RotaryEmbedding
    r = torch.load(os.path.join(golden_dir, "rope.pt"))
    rope = RotaryEmbedding(64, 64, 512, 1e6).to(DEV)
    assert torch.allclose(rope.cos_sin_cache.cpu(), r["cache"], rtol=0, atol=1e-6)
    rope.cos_sin_cache.copy_(r["cache"])  # the fixture's table, bit for bit
    q, k = r["q"].to(DEV), r["k"].to(DEV)
    q_in, k_in = q.clone(), k.clone()
    q_out, k_out = rope(r["pos"].to(DEV), q, k)
    torch.cuda.synchronize()
    assert torch.equal(q_out.cpu(), r["q_out"]) and torch.equal(k_out.cpu(), r["k_out"])
    assert torch.equal(q, q_in) and torch.equal(k, k_in)  # inputs untouched, as in the reference


def test_embedding_local(ops, golden_dir):
    d = torch.load(os.path.join(golden_dir, "vocab.pt"))
    got = ops.embed(d["ids"].to(DEV), d["w"].to(DEV), 0, d["w"].shape[0], 1)
    assert torch.equal(got.cpu(), d["emb"])
    w = torch.randn(1000, 4096).bfloat16()
    ids = torch.randint(0, 1000, (4, 33))
    assert torch.equal(ops.embed(ids.to(DEV), w.to(DEV), 0, 1000, 1).cpu(), w[ids])


def test_argmax(ops):
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(64, 151936, generator=g).bfloat16()
    logits[3, 77] = 50.0
    logits[3, 99] = 50.0  # tie: first index wins
    got = ops.argmax(logits.to(DEV)).cpu()
    assert torch.equal(got, logits.float().argmax(-1))
    assert got[3].item() == 77
    small = torch.randn(5, 1000, generator=g).bfloat16()
    assert torch.equal(ops.argmax(small.to(DEV)).cpu(), small.float().argmax(-1))
