"""Microbenchmark of the fused row-parallel block (GEMM + cross-GPU reduction +
residual add + RMSNorm in one launch) next to the reference's formulation of
the same block on the same GPUs: F.linear, NCCL all_reduce
(nanovllm/layers/linear.py:153-155) and the torch.compile'd add + RMSNorm
(nanovllm/layers/layernorm.py:28-40).

Both sides run inside CUDA graphs, as the decode path does, over a rotation of
weight copies larger than L2, and are timed with CUDA events (max over ranks).

Stand-alone, under torchrun with N ranks, it runs the Qwen3-32B shapes
(hidden 5120; o_proj K = 8192, down_proj K = 25600, split over N) for
M in {1, 8, 64, 256, 1024, 8192} and prints one JSON row per case:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        nano-vllm_b200/rowpar_microbench.py [--tokens 1,8,64] [--no-nccl]
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)


def roofline_us(m: int, n: int, kr: int, world: int, peaks: dict) -> dict:
    flops = 2.0 * m * n * kr
    nvl = 2.0 * (world - 1) / world * m * n * 2
    hbm = 2.0 * (m * kr + n * kr + 3 * m * n + n)
    t = {"flops_us": flops / (peaks["bf16_tflops"] * 1e12) * 1e6, "nvlink_us": nvl / (NVLINK_GBS * 1e9) * 1e6,
         "hbm_us": hbm / (peaks["hbm_gbs"] * 1e9) * 1e6}
    t["roof_us"] = max(t["flops_us"], t["nvlink_us"], t["hbm_us"])
    t["roof2_us"] = max(t["flops_us"], t["nvlink_us"])  # "the slower of compute at peak and bytes over NVLink"
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


def _reference_add_rms(x, residual, weight, eps):
    orig = x.dtype
    x = x.float().add_(residual.float())
    residual = x.to(orig)
    var = x.pow(2).mean(dim=-1, keepdim=True)
    x.mul_(torch.rsqrt(var + eps))
    return x.to(orig).mul_(weight), residual


def compare_blocks(blocks, peaks: dict, iters: int = 200, with_nccl: bool = True) -> dict:
    from . import ops
    world = dist.get_world_size() if dist.is_initialized() else 1
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    norm_fn = _reference_add_rms
    if with_nccl:
        try:
            norm_fn = torch.compile(_reference_add_rms)
        except Exception:
            norm_fn = _reference_add_rms
    for name, m, n, kr in blocks:
        n_w = int(max(2, min(64, (300 << 20) // (n * kr * 2) + 1)))
        ws = [(torch.randn(n, kr, device=dev) * 0.02).bfloat16() for _ in range(n_w)]
        x = torch.randn(m, kr, device=dev).bfloat16()
        residual = torch.randn(m, n, device=dev).bfloat16()
        norm_w = (torch.rand(n, device=dev) + 0.5).bfloat16()
        ours = time_in_graph(lambda i: ops.rowpar_fused(x, ws[i % n_w], None, residual, norm_w, 1e-6), n_w, iters)
        row = {"M": m, "N": n, "Kr": kr, "tp": world, "b200_us": ours}
        row.update(roofline_us(m, n, kr, world, peaks))
        row["frac_of_roof"] = row["roof_us"] / ours
        if with_nccl and world > 1:
            def ref_call(i):
                y = F.linear(x, ws[i % n_w])
                dist.all_reduce(y)
                return norm_fn(y, residual, norm_w, 1e-6)
            try:
                row["nccl_us"] = time_in_graph(ref_call, n_w, iters)
                row["speedup_vs_nccl"] = row["nccl_us"] / ours
            except Exception as ex:
                row["nccl_error"] = repr(ex)[:160]
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
    from .utils.context import set_context, reset_context
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
        rms, add_rms, rope, silu_mul = (torch.compile(f) for f in (_rms, lambda x, r, w: _reference_add_rms(x, r, w, eps), _rope, _silu_mul))
    except Exception:
        rms, add_rms, rope, silu_mul = _rms, (lambda x, r, w: _reference_add_rms(x, r, w, eps)), _rope, _silu_mul

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


TRACE_PHASES = ["set-up done", "first operand tile landed", "last MMA issued", "earlier kernels complete", "epilogue done",
                "GEMM part left", "reduce phase done", "kernel entry"]


def trace_phases(make_call, warmup: int = 3) -> dict:
    """Phase stamps of one launch of the fused block on this rank (the library's b2_trace): for every phase the
    minimum, median and maximum over the CTAs, in microseconds after the first CTA entered the kernel.  Each GPU
    has its own clock, so only the differences inside one rank mean something."""
    import ctypes as C

    import numpy as np

    from . import _abi
    from .runtime import get_runtime
    rt = get_runtime()
    for i in range(warmup):
        make_call(i)
    torch.cuda.synchronize()
    _abi.check(_abi.lib.b2_trace(rt.ctx, 1, None, 0), "b2_trace on")
    make_call(warmup)
    torch.cuda.synchronize()
    max_ctas = 256
    buf = (C.c_ulonglong * (max_ctas * 16))()
    _abi.check(_abi.lib.b2_trace(rt.ctx, 0, buf, max_ctas), "b2_trace read")
    ns = np.frombuffer(buf, dtype=np.uint64).reshape(max_ctas, 8, 2)[:, :, 1].astype(np.int64)
    live = ns[:, 7] > 0
    out = {"ctas": int(live.sum())}
    if not live.any():
        return out
    t0 = ns[live, 7].min()
    for i in (7, 0, 3, 1, 2, 4, 5, 6):
        v = ns[live, i]
        v = v[v > 0]
        if len(v):
            r = (v - t0) / 1e3
            out[TRACE_PHASES[i]] = [round(float(r.min()), 2), round(float(np.median(r)), 2), round(float(r.max()), 2)]
    return out


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
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--trace", action="store_true", help="instead of timing, print every rank's per-phase stamps of one launch per shape")
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
    init_runtime(max_tokens=max(ms), hidden=5120, oneshot_tokens=1024)
    try:
        for proj, k_total in (("o_proj", 8192), ("down_proj", 25600)):
            for m in ms:
                if a.trace:
                    from nanovllm_b200 import ops
                    kr = k_total // world
                    dev = torch.device("cuda", local)
                    ws = [(torch.randn(5120, kr, device=dev) * 0.02).bfloat16() for _ in range(4)]
                    x = torch.randn(m, kr, device=dev).bfloat16()
                    residual = torch.randn(m, 5120, device=dev).bfloat16()
                    norm_w = (torch.rand(5120, device=dev) + 0.5).bfloat16()
                    dist.barrier()
                    stamps = mb.trace_phases(lambda i: ops.rowpar_fused(x, ws[i % 4], None, residual, norm_w, 1e-6))
                    everyone = [None] * world
                    dist.all_gather_object(everyone, stamps)
                    if rank == 0:
                        for r, st in enumerate(everyone):
                            print(json.dumps({"proj": proj, "M": m, "Kr": kr, "tp": world, "rank": r} | st), flush=True)
                    continue
                res = mb.compare_blocks([(proj, m, 5120, k_total // world)], peaks, iters=a.iters if m <= 1024 else 20, with_nccl=not a.no_nccl)
                if rank == 0:
                    print(json.dumps(res[proj] | {"proj": proj}), flush=True)
    finally:
        shutdown_runtime()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
