"""The tcgen05 GEMM, the fused row-parallel launch and the LM head on one B200,
against the CPU oracle and the golden fixtures."""
import os

import pytest
import torch

from oracle import tp_path as O
from tests.gpu_util import assert_close_bf16, ensure_group, ulp_mismatch_fraction

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def rt(pkg):
    ensure_group()
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    r = init_runtime(max_tokens=16384, hidden=5120, oneshot_tokens=1024, vocab=151936, max_seqs=64)
    yield r
    shutdown_runtime()


@pytest.fixture(scope="module")
def ops(rt):
    from nanovllm_b200 import ops as _ops
    return _ops


def _case(m, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    return x, w


GEMM_SHAPES = [
    (64, 128, 64), (64, 128, 512), (1, 128, 256), (8, 256, 1024), (17, 384, 320), (64, 4096, 4096), (64, 6144, 4096),
    (33, 1000, 1024), (128, 1024, 1024), (200, 512, 768), (256, 2048, 1024), (257, 1024, 512), (1024, 5120, 1024), (1000, 1032, 520),
    (2048, 4096, 4096),
]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
def test_gemm_against_fp32(ops, rt, m, n, k):
    x, w = _case(m, n, k, m + n + k)
    got = ops.gemm(x.to(DEV), w.to(DEV))
    torch.cuda.synchronize()
    rt.check_status()
    ref = x.float() @ w.float().t()
    assert_close_bf16(got, ref, f"gemm {m}x{n}x{k}")
    # one rounding of an fp32 accumulation: at most 1 ulp from the oracle's rounding
    assert ulp_mismatch_fraction(got, O.linear(x, w), 1) < 1e-3


def test_gemm_bias_and_strided_input(ops, rt):
    x, w = _case(48, 512, 256, 5)
    bias = torch.randn(512).bfloat16()
    got = ops.gemm(x.to(DEV), w.to(DEV), bias.to(DEV))
    assert_close_bf16(got, x.float() @ w.float().t() + bias.float(), "gemm+bias (few tokens)")
    x2, w2 = _case(300, 512, 256, 6)
    got = ops.gemm(x2.to(DEV), w2.to(DEV), bias.to(DEV))
    assert_close_bf16(got, x2.float() @ w2.float().t() + bias.float(), "gemm+bias (many tokens)")
    wide = torch.randn(48, 1024).bfloat16().to(DEV)
    view = wide[:, 512:768]  # row stride 1024, offset 512 elements
    assert_close_bf16(ops.gemm(view, w.to(DEV)), view.float().cpu() @ w.float().t(), "gemm strided input")


def test_gemm_repeatable_and_counters_clean(ops, rt):
    """Split tiles are combined through arrival counters that must be back at
    zero after every launch: the same call twice gives the same result (up to
    the order in which the fp32 partials of a tile are added, which depends on
    which CTA arrives last)."""
    x, w = _case(64, 4096, 12288, 9)
    a = ops.gemm(x.to(DEV), w.to(DEV))
    b = ops.gemm(x.to(DEV), w.to(DEV))
    torch.cuda.synchronize()
    assert_close_bf16(a, x.float() @ w.float().t(), "gemm 64x4096x12288")
    assert_close_bf16(b, a.float(), "second launch", abs_tol=2e-3, rel_tol=8e-3)  # at most one bf16 ulp apart


@pytest.mark.parametrize("m,i,k", [(64, 12288, 4096), (64, 1536, 4096), (7, 256, 512), (300, 1024, 1024), (1100, 3072, 1024)])
def test_gemm_silu_mul(ops, rt, m, i, k):
    """gate_up GEMM with SiLU * mul in the epilogue against gemm followed by the oracle's activation."""
    g = torch.Generator().manual_seed(m + i)
    x = torch.randn(m, k, generator=g).bfloat16()
    wg = (torch.randn(i, k, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(i, k, generator=g) * 0.05).bfloat16()
    pairs = torch.stack((wg, wu), dim=1).reshape(2 * i, k).contiguous()
    got = ops.gemm_silu_mul(x.to(DEV), pairs.to(DEV))
    torch.cuda.synchronize()
    rt.check_status()
    ref = O.silu_and_mul(torch.cat([O.linear(x, wg), O.linear(x, wu)], dim=-1))
    exact = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    assert_close_bf16(got, exact, f"gemm_silu_mul {m}x{i}x{k}", abs_tol=3e-2, rel_tol=2e-2)
    assert ulp_mismatch_fraction(got, ref, 2) < 2e-2  # same roundings as the two-kernel form, up to the GEMM's own last-bit differences


@pytest.mark.parametrize("m,nq,nkv,k", [(64, 32, 8, 4096), (64, 4, 1, 4096), (9, 4, 2, 512), (300, 4, 2, 512)])
def test_qkv_fused_matches_two_kernel_form(ops, rt, m, nq, nkv, k):
    """Projection + head norm + RoPE + KV scatter in one call against gemm followed by the head kernel."""
    hd = 128
    g = torch.Generator().manual_seed(m + nq)
    x = torch.randn(m, k, generator=g).bfloat16().to(DEV)
    w = (torch.randn((nq + 2 * nkv) * hd, k, generator=g) * 0.05).bfloat16().to(DEV)
    qw = (torch.rand(hd, generator=g) + 0.5).bfloat16().to(DEV)
    kw = (torch.rand(hd, generator=g) + 0.5).bfloat16().to(DEV)
    pos = torch.randint(0, 512, (m,), generator=g).to(DEV)
    cache = O.rope_cache(hd, 512, 1e6).to(DEV)
    slots = torch.randperm(4 * 256, generator=g)[:m].to(torch.int32)
    slots[::7] = -1
    slots = slots.to(DEV)
    kc1 = torch.zeros(4, 256, nkv, hd, dtype=torch.bfloat16, device=DEV)
    vc1, kc2, vc2 = torch.zeros_like(kc1), torch.zeros_like(kc1), torch.zeros_like(kc1)
    fused = ops.qkv_fused(x, w, None, nq, nkv, hd, qw, kw, 1e-6, pos, cache, kc1, vc1, slots)
    two = ops.gemm(x, w)
    ops.qk_norm_rope_store(two, nq, nkv, hd, qw, kw, 1e-6, pos, cache, kc2, vc2, slots)
    torch.cuda.synchronize()
    rt.check_status()
    assert torch.equal(fused, two)
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    # and against the oracle's statement of the same steps
    y = O.linear(x.cpu(), w.cpu())
    q, kk, v = y.split([nq * hd, nkv * hd, nkv * hd], dim=-1)
    q_ref = O.apply_rope(O.rms_norm(q.reshape(m, nq, hd), qw.cpu(), 1e-6), pos.cpu(), cache.cpu())
    assert ulp_mismatch_fraction(fused[:, :nq * hd].cpu().reshape(m, nq, hd), q_ref, 2) < 2e-2


@pytest.mark.parametrize("paired", [False, True])
def test_merged_column_layer_paired_weight(pkg, rt, golden_dir, paired):
    from nanovllm_b200.layers.linear import MergedColumnParallelLinear
    d = torch.load(os.path.join(golden_dir, "col.pt"))
    torch.set_default_dtype(torch.bfloat16)
    try:
        layer = MergedColumnParallelLinear(128, [192 * 1, 192 * 1]).to(DEV)  # world 1: both halves whole
    finally:
        torch.set_default_dtype(torch.float32)
    if paired:
        layer.pair_rows()  # rows interleaved by the loader: no second copy of the weight
    layer.weight.weight_loader(layer.weight, d["wg"].to(DEV), 0)
    layer.weight.weight_loader(layer.weight, d["wu"].to(DEV), 1)
    assert torch.equal(layer.reference_weight().cpu(), torch.cat((d["wg"], d["wu"])))
    if paired:
        assert layer.paired_weight().data_ptr() == layer.weight.data_ptr()
    x = d["x"].to(DEV)
    y = layer(x)
    assert ulp_mismatch_fraction(y, O.linear(d["x"], torch.cat((d["wg"], d["wu"]))), 1) < 2e-3
    act = layer.forward_silu_mul(x)
    assert ulp_mismatch_fraction(act, O.silu_and_mul(y.cpu()), 2) < 2e-2


def test_column_parallel_golden(ops, golden_dir):
    d = torch.load(os.path.join(golden_dir, "col.pt"))
    for r in range(2):
        yq = ops.gemm(d["x"].to(DEV), d[f"qkv_w{r}"].to(DEV))
        yg = ops.gemm(d["x"].to(DEV), d[f"gu_w{r}"].to(DEV))
        assert ulp_mismatch_fraction(yq, d[f"qkv_y{r}"], 1) < 2e-3
        assert ulp_mismatch_fraction(yg, d[f"gu_y{r}"], 1) < 2e-3


ROWPAR_SHAPES = [(64, 2048, 1024), (64, 3072, 1024), (1, 4096, 4096), (8, 12288, 4096), (64, 4096, 4096), (64, 12288, 4096),
                 (256, 8192, 5120), (300, 1024, 5120), (1024, 1024, 5120), (1500, 512, 1024)]


@pytest.mark.parametrize("m,k,n", ROWPAR_SHAPES)
def test_rowpar_fused_single_rank(ops, rt, m, k, n):
    xs, ws, residual, norm_w = O.rowpar_case(m, k, n, 1, seed=m + k)
    for _ in range(3):  # consecutive launches alternate between the two inboxes
        normed, new_res = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
    torch.cuda.synchronize()
    rt.check_status()
    exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
    assert_close_bf16(new_res, exact_s, f"residual {m}x{k}x{n}")
    assert_close_bf16(normed, exact_n, f"normed {m}x{k}x{n}")
    ref_n, ref_s = O.fused_row_parallel_norm(xs, ws, residual, norm_w, 1e-6)
    assert ulp_mismatch_fraction(new_res, ref_s, 1) < 2e-3
    assert ulp_mismatch_fraction(normed, ref_n, 2) < 2e-3


OWNER_SHAPES = [(64, 2048, 1024), (1, 4096, 4096), (8, 12288, 4096), (64, 4096, 4096), (5, 1024, 5120), (63, 512, 4096),
                (65, 1024, 5120), (256, 8192, 5120), (300, 1024, 5120), (1024, 1024, 5120), (1500, 512, 1024)]


@pytest.mark.parametrize("m,k,n", OWNER_SHAPES)
def test_rowpar_owner_form_single_rank(ops, rt, m, k, n):
    """The row-owner form of the fused block (partial rows to the owner's inbox, finished rows into the landing
    buffer, collected into the caller's tensors), forced on one rank, where rank 0 owns every row: same outputs as
    the one-shot form."""
    from nanovllm_b200 import _abi
    xs, ws, residual, norm_w = O.rowpar_case(m, k, n, 1, seed=m + k)
    one_n, one_s = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
    rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_OWNER)
    try:
        assert ops.rowpar_form(min(m, 1024), n) == _abi.FORM_OWNER
        for i in range(3):  # consecutive launches alternate between the two inboxes / landing buffers
            normed, new_res = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
        y = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, None, None, 0.0)  # plain forward through the same form
        torch.cuda.synchronize()
        rt.check_status()
    finally:
        rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
    exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
    assert_close_bf16(new_res, exact_s, f"owner form residual {m}x{k}x{n}")
    assert_close_bf16(normed, exact_n, f"owner form normed {m}x{k}x{n}")
    assert_close_bf16(y, xs[0].float() @ ws[0].float().t(), f"owner form plain forward {m}x{k}x{n}")
    if m <= 64:  # both forms run the same (deterministic) cluster GEMM: identical values
        assert torch.equal(normed, one_n) and torch.equal(new_res, one_s)
    # mixing the forms launch by launch keeps the two inbox parities in step
    for i in range(4):
        rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_OWNER if i % 2 else _abi.FORM_ONESHOT)
        normed, new_res = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
    rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
    torch.cuda.synchronize()
    rt.check_status()
    assert_close_bf16(normed, exact_n, f"alternating forms {m}x{k}x{n}")


@pytest.mark.parametrize("m,k,n", [(128, 2048, 1024), (256, 1024, 2048), (200, 512, 1024), (96, 3072, 1024)])
def test_rowpar_oneshot_token_tiles_single_rank(ops, rt, m, k, n):
    """65..256 tokens through the one-shot form on the cluster kernel's 64-token tiles (what 2 and 4 ranks run at these
    sizes), forced on one rank, where the default would be the plain GEMM followed by the norm kernel."""
    from nanovllm_b200 import _abi
    xs, ws, residual, norm_w = O.rowpar_case(m, k, n, 1, seed=m + k + 1)
    auto_n, auto_s = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
    rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_ONESHOT)
    try:
        for _ in range(3):
            normed, new_res = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), None, residual.to(DEV), norm_w.to(DEV), 1e-6)
        assert _abi.lib.b2_last_gemm_kernel() == 1, "expected the cluster kernel"
        torch.cuda.synchronize()
        rt.check_status()
    finally:
        rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
    exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
    assert_close_bf16(new_res, exact_s, f"one-shot token tiles residual {m}x{k}x{n}")
    assert_close_bf16(normed, exact_n, f"one-shot token tiles normed {m}x{k}x{n}")
    assert_close_bf16(auto_n, exact_n, f"GEMM + norm kernel normed {m}x{k}x{n}")
    assert_close_bf16(auto_s, exact_s, f"GEMM + norm kernel residual {m}x{k}x{n}")


def test_rowpar_plain_forward_and_bias(ops, rt):
    """norm_w = None is RowParallelLinear.forward: y = x W^T (+ bias)."""
    xs, ws, _, _ = O.rowpar_case(64, 1024, 1024, 1, seed=4)
    bias = torch.randn(1024).bfloat16()
    y = ops.rowpar_fused(xs[0].to(DEV), ws[0].to(DEV), bias.to(DEV), None, None, 0.0)
    assert_close_bf16(y, xs[0].float() @ ws[0].float().t() + bias.float(), "row-parallel forward + bias")


def test_rowpar_golden(ops, rt, golden_dir):
    """The reference's TP=2 block outputs, reproduced on one rank holding the
    whole K (the only difference is where the partials are rounded)."""
    for name in ("rp_a", "rp_b"):
        d = torch.load(os.path.join(golden_dir, name + ".pt"))
        normed, new_res = ops.rowpar_fused(d["x_full"].to(DEV), d["w_full"].to(DEV), None, d["residual"].to(DEV), d["norm_w"].to(DEV), 1e-6)
        assert_close_bf16(new_res, d["new_res"].float(), name + " residual")
        assert_close_bf16(normed, d["normed"].float(), name + " normed")


def test_lm_head_single_rank(ops, rt):
    g = torch.Generator().manual_seed(2)
    h = torch.randn(40, 1024, generator=g).bfloat16()
    w = (torch.randn(151936, 1024, generator=g) * 0.02).bfloat16()
    logits = ops.lm_head(h.to(DEV), w.to(DEV), None)
    torch.cuda.synchronize()
    assert logits.shape == (40, 151936)
    assert_close_bf16(logits, h.float() @ w.float().t(), "lm_head decode")
    idx = torch.tensor([4, 5, 16, 39], dtype=torch.int32)
    logits = ops.lm_head(h.to(DEV), w.to(DEV), idx.to(DEV))
    torch.cuda.synchronize()
    assert logits.shape == (4, 151936)
    assert_close_bf16(logits, h[idx.long()].float() @ w.float().t(), "lm_head prefill (last tokens)")
    assert torch.equal(ops.argmax(logits).cpu(), logits.float().argmax(-1).cpu())


PAIR_SCRIPT = r"""
import sys, torch
sys.path.insert(0, %(root)r)
import __graft_entry__ as entry
entry.load_package()
from tests.gpu_util import assert_close_bf16, ensure_group
ensure_group()
from nanovllm_b200 import ops, _abi
from nanovllm_b200.runtime import init_runtime, shutdown_runtime
rt = init_runtime(max_tokens=8192, hidden=5120, oneshot_tokens=1024, timeout_ms=2000)
for (m, n, k) in [(512, 256, 64), (512, 512, 256), (1000, 1032, 520), (1024, 5120, 1024), (777, 128, 1024), (4096, 4096, 4096)]:
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    y = ops.gemm(x.cuda(), w.cuda())
    used = _abi.lib.b2_last_gemm_kernel()
    torch.cuda.synchronize()
    rt.check_status()
    assert used == 2, (m, n, k, used)
    assert_close_bf16(y, x.float() @ w.float().t(), f"pair gemm {m}x{n}x{k}")
    print("ok", m, n, k, flush=True)
shutdown_runtime()
"""


def test_pair_kernel():
    """The tcgen05.mma.cta_group::2 kernel (the default from 512 tokens on), in a child process of its own."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_PORT="29547")
    env.pop("B2_PAIR", None)
    res = subprocess.run([sys.executable, "-c", PAIR_SCRIPT % {"root": root}], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
