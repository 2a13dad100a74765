"""Microbenchmark of the fused row-parallel block (GEMM + cross-GPU reduction +
residual add + RMSNorm in one launch) next to the reference's own modules for
the same block on the same GPUs: RowParallelLinear (F.linear + NCCL
all_reduce, nanovllm/layers/linear.py:131-156) followed by RMSNorm's
add_rms_forward (torch.compile'd, nanovllm/layers/layernorm.py:28-40),
imported from the reference's install under baseline/_ref when it is there
(a restatement of the same calls otherwise; the JSON says which).

Both sides run inside CUDA graphs, as the decode path does, over a rotation of
weight copies larger than L2, and are timed with CUDA events (max over ranks).
After the timing one more call of each side runs on the same tensors and the
outputs are compared: ours against an fp32 statement of the block (per element,
|err| <= 2e-2 + 1e-2 |ref|) and against the reference modules' bf16 result.

Stand-alone, under torchrun with N ranks, it runs the Qwen3-32B shapes
(hidden 5120; o_proj K = 8192, down_proj K = 25600, split over N) for
M in {1, 8, 64, 256, 1024, 8192} and prints one JSON row per case:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        nano-vllm_b200/rowpar_microbench.py [--tokens 1,8,64] [--no-nccl] [--forms]
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

# Peer-copy bandwidth per direction per GPU through NVSwitch used as the NVLink term of the roofline (nominal
# 900 GB/s); the stand-alone run measures the copy itself and prints it beside every row.
NVLINK_GBS = 770.0
NVLINK_NOMINAL_GBS = 900.0
TOL_ABS, TOL_REL = 2e-2, 1e-2


def roofline_us(m: int, n: int, kr: int, world: int, peaks: dict) -> dict:
    flops = 2.0 * m * n * kr
    nvl = 2.0 * (world - 1) / world * m * n * 2
    hbm = 2.0 * (m * kr + n * kr + 3 * m * n + n)
    t = {"flops_us": flops / (peaks["bf16_tflops"] * 1e12) * 1e6, "nvlink_us": nvl / (NVLINK_GBS * 1e9) * 1e6,
         "hbm_us": hbm / (peaks["hbm_gbs"] * 1e9) * 1e6, "nvlink_bytes": nvl}
    t["roof_us"] = max(t["flops_us"], t["nvlink_us"], t["hbm_us"])
    t["roof2_us"] = max(t["flops_us"], t["nvlink_us"])  # "the slower of compute at peak and bytes over NVLink"
    t["roof_us_nominal_nvlink"] = max(t["flops_us"], nvl / (NVLINK_NOMINAL_GBS * 1e9) * 1e6, t["hbm_us"])
    return t


def _max_over_ranks(v: float) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_in_graph(make_call, n_variants: int, iters: int) -> float:
    """make_call(i) issues the i-th variant of the call on the current stream.
    One CUDA graph holds n_variants calls; returns microseconds per call."""
    for i in range(min(n_variants, 3)):
        make_call(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n_variants):
            make_call(i)
    replays = max(1, iters // n_variants)
    graph.replay()
    torch.cuda.synchronize()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return _max_over_ranks(e0.elapsed_time(e1) * 1e3 / (replays * n_variants))


def _restated_add_rms(x, residual, weight, eps):
    orig = x.dtype
    x = x.float().add_(residual.float())
    residual = x.to(orig)
    var = x.pow(2).mean(dim=-1, keepdim=True)
    x.mul_(torch.rsqrt(var + eps))
    return x.to(orig).mul_(weight), residual


def reference_install() -> str | None:
    """Directory of the reference's install (baseline/_ref beside the package), or None."""
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(os.path.dirname(here), "baseline", "_ref")
    return path if os.path.isdir(os.path.join(path, "nanovllm")) else None


class ReferenceBlock:
    """The reference's formulation of the block on this rank's GPU: its own RowParallelLinear and RMSNorm modules
    when the install is present (`kind` = "reference modules"), the same calls restated otherwise."""

    def __init__(self, n: int, k_total: int, kr: int, norm_w: torch.Tensor, eps: float, dev):
        self.kind = "restated calls (F.linear + dist.all_reduce + torch.compile'd add-RMSNorm)"
        self.linear = self.norm = None
        self.norm_w, self.eps = norm_w, eps
        path = reference_install()
        if path is not None and dist.is_initialized():
            try:
                if path not in sys.path:
                    sys.path.insert(0, path)
                from nanovllm.layers.layernorm import RMSNorm
                from nanovllm.layers.linear import RowParallelLinear
                prev = torch.get_default_dtype()
                torch.set_default_dtype(torch.bfloat16)
                try:
                    with torch.device(dev):
                        self.linear = RowParallelLinear(k_total, n, bias=False)
                        self.norm = RMSNorm(n, eps=eps)
                finally:
                    torch.set_default_dtype(prev)
                assert tuple(self.linear.weight.shape) == (n, kr)
                self.norm.weight.data.copy_(norm_w)
                self.kind = "reference modules (nanovllm RowParallelLinear + RMSNorm, NCCL all_reduce)"
            except Exception as ex:  # fall back to the restated calls, and say why
                self.linear = self.norm = None
                self.kind += f" [reference import failed: {ex!r}]"[:200]
        if self.linear is None:
            try:
                self._add_rms = torch.compile(_restated_add_rms)
            except Exception:
                self._add_rms = _restated_add_rms

    @torch.inference_mode()  # as the reference runs its model (nanovllm/engine/model_runner.py:195)
    def __call__(self, x, w, residual):
        if self.linear is not None:
            self.linear.weight.data = w
            return self.norm(self.linear(x), residual)
        y = F.linear(x, w)
        if dist.get_world_size() > 1:
            dist.all_reduce(y)
        return self._add_rms(y, residual, self.norm_w, self.eps)


def _error_stats(got: torch.Tensor, ref: torch.Tensor, unit_scale: bool = True) -> dict:
    """Per element |err| <= abs + rel |ref|.  abs = 2e-2 for unit-scale rows (the normalised output); for the
    un-normalised residual sum, whose size grows with K, abs = 2e-2 x the row's RMS (when that exceeds 1): the bf16
    partial products that cross NVLink carry half a unit in the last place of THEIR size even where they cancel."""
    got, ref = got.float(), ref.float()
    err = (got - ref).abs()
    big = ref.abs() >= 1.0
    scale = 1.0 if unit_scale else ref.pow(2).mean(-1, keepdim=True).sqrt().clamp_min(1.0)
    return {"max_abs_err": err.max().item(), "max_rel_err": (err[big] / ref.abs()[big]).max().item() if bool(big.any()) else 0.0,
            "within_tolerance": bool((err <= TOL_ABS * scale + TOL_REL * ref.abs()).all())}


def compare_blocks(blocks, peaks: dict, iters: int = 200, with_nccl: bool = True, forms: bool = False) -> dict:
    """blocks: (name, M, N, Kr) per case.  Returns per case the timings, the roofline and the parity of the last call.
    forms=True also times b2_rowpar_fused with each of its two forms forced (one-shot, row-owner)."""
    from . import _abi, ops
    from .runtime import get_runtime
    rt = get_runtime()
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    for name, m, n, kr in blocks:
        n_w = int(max(2, min(64, (300 << 20) // (n * kr * 2) + 1)))
        g_own = torch.Generator(device=dev).manual_seed(1000 + 17 * rank + m + kr)   # this rank's shard of the operands
        g_all = torch.Generator(device=dev).manual_seed(77 + m + n)                  # what every rank holds alike
        ws = [(torch.randn(n, kr, device=dev, generator=g_own) * 0.02).bfloat16() for _ in range(n_w)]
        x = torch.randn(m, kr, device=dev, generator=g_own).bfloat16()
        residual = torch.randn(m, n, device=dev, generator=g_all).bfloat16()
        norm_w = (torch.rand(n, device=dev, generator=g_all) + 0.5).bfloat16()

        def ours_call(i):
            return ops.rowpar_fused(x, ws[i % n_w], None, residual, norm_w, 1e-6)

        def timed(label):
            """One timing; an expired device-side wait is reported in the row and the context reset on every rank."""
            us = time_in_graph(ours_call, n_w, iters)
            flag = torch.zeros(1, dtype=torch.int32)
            try:
                rt.check_status()
            except _abi.B2Error as ex:
                flag[0] = 1
                row.setdefault("errors", {})[label] = str(ex)
            if world > 1:
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            if flag.item():
                row.setdefault("errors", {}).setdefault(label, "a wait expired on another rank")
                rt.poisoned = True
                rt.reset()
            return us

        form = ops.rowpar_form(m, n)
        row = {}
        ours = timed("auto")
        row.update({"M": m, "N": n, "Kr": kr, "tp": world, "b200_us": ours,
                    "form": {_abi.FORM_ONESHOT: "one-shot", _abi.FORM_OWNER: "row-owner", _abi.FORM_TWOSHOT: "two-shot"}[form]})
        if forms and world > 1 and m <= rt.oneshot_tokens:
            rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, 1 << 30)
            for f, label in ((_abi.FORM_ONESHOT, "oneshot_us"), (_abi.FORM_OWNER, "owner_us")):
                rt.set_option(_abi.OPT_ROWPAR_FORM, f)
                row[label] = timed(label)
            if m > 64:  # token-row layout: with the stream-K split instead of one whole tile per CTA
                rt.set_option(_abi.OPT_WHOLE_TILES, 0)
                row["owner_streamk_us"] = timed("owner_streamk_us")
                rt.set_option(_abi.OPT_WHOLE_TILES, 1)
            rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
            if n == rt.hidden and m >= 16:
                rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, 1)
                row["twoshot_us"] = timed("twoshot_us")
            rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, rt.default_twoshot_min_tokens)
        row.update(roofline_us(m, n, kr, world, peaks))
        row["frac_of_roof"] = row["roof_us"] / ours
        row["nvlink_egress_gbs"] = row["nvlink_bytes"] / (ours * 1e-6) / 1e9 if world > 1 else 0.0
        # ---- parity of one more call on the first weight copy ----
        normed, new_res = ours_call(0)
        normed = normed.clone()
        y32 = x.float() @ ws[0].float().t()
        if world > 1:
            dist.all_reduce(y32)  # fp32 sum over the ranks: the exact block
        s = y32 + residual.float()
        exact = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.float()
        row["parity_vs_fp32"] = _error_stats(normed, exact)
        if form != _abi.FORM_TWOSHOT:  # (the two-shot form keeps the residual row-sharded)
            row["parity_vs_fp32"]["residual_within_tolerance"] = _error_stats(new_res, s, unit_scale=False)["within_tolerance"]
        if with_nccl and world > 1:
            try:
                ref = ReferenceBlock(n, kr * world, kr, norm_w, 1e-6, dev)
                row["reference_kind"] = ref.kind
                row["nccl_us"] = time_in_graph(lambda i: ref(x, ws[i % n_w], residual), n_w, iters)
                row["speedup_vs_nccl"] = row["nccl_us"] / ours
                ref_n, _ = ref(x.clone(), ws[0], residual.clone())
                row["parity_vs_reference"] = {"max_abs_diff": (normed.float() - ref_n.float()).abs().max().item(),
                                              "reference_vs_fp32": _error_stats(ref_n, exact)}
            except Exception as ex:
                row["nccl_error"] = repr(ex)[:200]
        out[name] = row
        del ws
        torch.cuda.empty_cache()
    return out


def compare_model_forward(runner, bs: int, iters: int = 20) -> dict:
    """One decode forward pass of the runner's model (all decoder layers, batch `bs`) in two forms, each in
    its own CUDA graph on the same weights, KV cache and batch state:
      ours      - the runner's captured graph (fused kernels of this library)
      reference - the reference's formulation of the same pass: F.linear for every projection
                  (nanovllm/layers/linear.py:73,153), NCCL all_reduce after o_proj and down_proj (:155),
                  torch.compile'd RMSNorm / add+RMSNorm / RoPE / SiLU*mul (nanovllm/layers/layernorm.py,
                  rotary_embedding.py, activation.py), an index_copy_ for the KV scatter, and the same
                  flash-attn decode call (nanovllm/layers/attention.py:72-74).
    Returns microseconds per pass (max over ranks)."""
    from flash_attn import flash_attn_with_kvcache
    world = dist.get_world_size() if dist.is_initialized() else 1
    model = runner.model.model
    gv = runner.graph_vars
    eps = runner.config.rms_norm_eps

    def _rms(x, w):
        dt = x.dtype
        x = x.float()
        var = x.pow(2).mean(dim=-1, keepdim=True)
        x.mul_(torch.rsqrt(var + eps))
        return x.to(dt).mul_(w)

    def _rope(cos_sin, q, k):
        cos, sin = cos_sin.chunk(2, dim=-1)

        def rot(x):
            x1, x2 = torch.chunk(x.float(), 2, dim=-1)
            return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1).to(x.dtype)
        return rot(q), rot(k)

    def _silu_mul(x):  # the model stores gate and up rows interleaved: columns come out as (gate_0, up_0, gate_1, ...)
        return F.silu(x[..., 0::2]) * x[..., 1::2]

    try:
        rms, add_rms, rope, silu_mul = (torch.compile(f) for f in (_rms, lambda x, r, w: _restated_add_rms(x, r, w, eps), _rope, _silu_mul))
    except Exception:
        rms, add_rms, rope, silu_mul = _rms, (lambda x, r, w: _restated_add_rms(x, r, w, eps)), _rope, _silu_mul

    @torch.inference_mode()
    def reference_pass():
        ids, pos = gv["input_ids"][:bs], gv["positions"][:bs]
        slots, lens, tables = gv["slot_mapping"][:bs].long(), gv["context_lens"][:bs], gv["block_tables"][:bs]
        emb = model.embed_tokens
        if world > 1:
            mask = (ids >= emb.vocab_start_idx) & (ids < emb.vocab_end_idx)
            h = F.embedding(mask * (ids - emb.vocab_start_idx), emb.weight) * mask.unsqueeze(1)
            dist.all_reduce(h)
        else:
            h = F.embedding(ids, emb.weight)
        residual = None
        y = h
        for layer in model.layers:
            att = layer.self_attn
            if residual is None:
                residual, h = y, rms(y, layer.input_layernorm.weight)
            else:
                h, residual = add_rms(y, residual, layer.input_layernorm.weight)
            qkv = F.linear(h, att.qkv_proj.weight)
            q, k, v = qkv.split([att.q_size, att.kv_size, att.kv_size], dim=-1)
            q = rms(q.view(-1, att.num_heads, att.head_dim), att.q_norm.weight)
            k = rms(k.view(-1, att.num_kv_heads, att.head_dim), att.k_norm.weight)
            q, k = rope(att.rotary_emb.cos_sin_cache[pos].unsqueeze(1), q, k)
            kc, vc = att.attn.k_cache, att.attn.v_cache
            kc.view(-1, att.num_kv_heads, att.head_dim).index_copy_(0, slots, k)
            vc.view(-1, att.num_kv_heads, att.head_dim).index_copy_(0, slots, v.view(-1, att.num_kv_heads, att.head_dim))
            o = flash_attn_with_kvcache(q.unsqueeze(1), kc, vc, cache_seqlens=lens, block_table=tables, softmax_scale=att.scaling, causal=True)
            y = F.linear(o.flatten(1, -1), att.o_proj.weight)
            if world > 1:
                dist.all_reduce(y)
            h, residual = add_rms(y, residual, layer.post_attention_layernorm.weight)
            act = silu_mul(F.linear(h, layer.mlp.gate_up_proj.weight))
            y = F.linear(act, layer.mlp.down_proj.weight)
            if world > 1:
                dist.all_reduce(y)
        out, _ = add_rms(y, residual, model.norm.weight)
        return out

    for _ in range(3):
        reference_pass()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        reference_pass()

    def timed(replay):
        replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            replay()
        e1.record()
        torch.cuda.synchronize()
        return _max_over_ranks(e0.elapsed_time(e1) * 1e3 / iters)

    ref_us = timed(graph.replay)
    ours_us = timed(runner.graphs[bs].replay)
    return {"b200_us": ours_us, "reference_formulation_nccl_us": ref_us, "speedup": ref_us / ours_us, "batch": bs, "tp": world,
            "what": "model forward only (embedding, all decoder layers, final norm); LM head and sampling excluded on both sides"}


def measure_peer_copy_gbs(local: int, world: int, mib: int = 512) -> float | None:
    """GB/s of a device-to-device copy from this rank's GPU to the next rank's, every rank copying at once
    (one direction of every GPU's NVLink ports busy): the figure the NVLink term of the roofline stands for."""
    if world < 2:
        return None
    try:
        src = torch.empty(mib << 20, dtype=torch.uint8, device=torch.device("cuda", local))
        dst = torch.empty(mib << 20, dtype=torch.uint8, device=torch.device("cuda", (local + 1) % world))
        for _ in range(2):
            dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(8):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        ms = _max_over_ranks(e0.elapsed_time(e1) / 8)
        del src, dst
        return (mib << 20) / (ms * 1e-3) / 1e9
    except Exception:
        return None


def main():
    import argparse
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(here))
    import __graft_entry__ as entry
    entry.load_package()
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    from nanovllm_b200 import rowpar_microbench as mb  # the package-relative copy of this module

    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,8,64,256,1024,8192")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--forms", action="store_true", help="also time b2_rowpar_fused with each of its forms forced")
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--shapes", default="32b", choices=["32b", "8b"], help="Qwen3-32B (hidden 5120) or Qwen3-8B (hidden 4096) projections")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl" if world > 1 else "gloo", rank=rank, world_size=world)
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    p = os.path.join(os.path.dirname(here), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        peaks = json.load(open(p))
    ms = [int(v) for v in a.tokens.split(",")]
    hidden, projections = (5120, (("o_proj", 8192), ("down_proj", 25600))) if a.shapes == "32b" else (4096, (("o_proj", 4096), ("down_proj", 12288)))
    peer_gbs = mb.measure_peer_copy_gbs(local, world)
    init_runtime(max_tokens=max(ms), hidden=hidden, oneshot_tokens=1024)
    try:
        for proj, k_total in projections:
            for m in ms:
                res = mb.compare_blocks([(proj, m, hidden, k_total // world)], peaks, iters=a.iters if m <= 1024 else 20, with_nccl=not a.no_nccl,
                                        forms=a.forms)
                if rank == 0:
                    print(json.dumps(res[proj] | {"proj": proj, "peer_copy_gbs_measured": peer_gbs}), flush=True)
    finally:
        shutdown_runtime()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
