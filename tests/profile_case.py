"""Run one kernel of the library a few times on one GPU, for profiling with
Nsight Compute (the cases are larger than the 126 MB L2 but hold well under a
few GB, so a `--set full` capture of 1-3 launches ends by itself).

    python tests/profile_case.py <case> [--launches 6]

cases:
  gemm_decode     column-parallel GEMM, M=64, N=24576, K=4096 (Qwen3-8B gate_up at TP=1), 4 weight copies
  silu_decode     the same GEMM with SiLU*mul in its epilogue (what the decoder layer launches)
  qkv_decode      qkv projection M=64, N=6144, K=4096 with q/k-norm + RoPE + KV scatter in its epilogue, 8 weight copies
  oproj_decode    fused row-parallel launch, M=64, N=4096, Kr=4096 (Qwen3-8B o_proj at TP=1), 8 weight copies
  gemm_prefill    GEMM M=4096, N=4096, K=4096
  gemm_mid        GEMM M=256, N=4096, K=1024 (Qwen3-0.6B qkv at a 256-sequence decode step), 40 weight copies
  rowpar_decode   fused row-parallel launch, M=64, N=4096, Kr=12288 (Qwen3-8B down_proj at TP=1)
  rowpar_prefill  fused row-parallel launch, M=1024, N=5120, Kr=1024
  store_kvcache   paged-KV scatter, 16384 tokens x D=1024
  add_rmsnorm     residual add + RMSNorm, 16384 x 4096
  embed           embedding lookup, 16384 ids into a [151936, 4096] table (one rank)
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--launches", type=int, default=6)
    a = ap.parse_args()
    import __graft_entry__ as entry
    entry.load_package()
    from nanovllm_b200 import ops
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29579")
    torch.cuda.set_device(0)
    dist.init_process_group("gloo", rank=0, world_size=1)
    init_runtime(max_tokens=16384, hidden=5120, oneshot_tokens=1024)
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).bfloat16()

    if a.case in ("gemm_decode", "gemm_prefill", "gemm_mid"):
        m, n, k, copies = {"gemm_decode": (64, 24576, 4096, 4), "gemm_prefill": (4096, 4096, 4096, 2), "gemm_mid": (256, 4096, 1024, 40)}[a.case]
        x, ws = rnd(m, k), [rnd(n, k, scale=0.02) for _ in range(copies)]
        call = lambda i: ops.gemm(x, ws[i % copies])
    elif a.case == "silu_decode":
        m, i, k, copies = 64, 12288, 4096, 4
        x, ws = rnd(m, k), [rnd(2 * i, k, scale=0.02) for _ in range(copies)]
        call = lambda j: ops.gemm_silu_mul(x, ws[j % copies])
    elif a.case == "qkv_decode":
        m, nq, nkv, k, copies = 64, 32, 8, 4096, 8
        x, ws = rnd(m, k), [rnd((nq + 2 * nkv) * 128, k, scale=0.02) for _ in range(copies)]
        qw, kw = rnd(128), rnd(128)
        pos = torch.randint(0, 2048, (m,), device=dev)
        t = torch.arange(2048, dtype=torch.float, device=dev)
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, dtype=torch.float, device=dev) / 128))
        fr = torch.outer(t, inv)
        cos_sin = torch.cat((fr.cos(), fr.sin()), dim=-1).contiguous()
        kc = torch.zeros(16, 256, nkv, 128, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        slots = torch.randperm(16 * 256, device=dev)[:m].to(torch.int32)
        call = lambda j: ops.qkv_fused(x, ws[j % copies], None, nq, nkv, 128, qw, kw, 1e-6, pos, cos_sin, kc, vc, slots)
    elif a.case in ("rowpar_decode", "rowpar_prefill", "oproj_decode"):
        m, n, k, copies = {"rowpar_decode": (64, 4096, 12288, 4), "rowpar_prefill": (1024, 5120, 1024, 8), "oproj_decode": (64, 4096, 4096, 8)}[a.case]
        x, ws, res, nw = rnd(m, k), [rnd(n, k, scale=0.02) for _ in range(copies)], rnd(m, n), rnd(n)
        call = lambda i: ops.rowpar_fused(x, ws[i % copies], None, res, nw, 1e-6)
    elif a.case == "store_kvcache":
        n, heads = 16384, 8
        key, value = rnd(n, heads, 128), rnd(n, heads, 128)
        kc = torch.zeros(2, 128, 256, heads, 128, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        perm = torch.randperm(128, device=dev, generator=g)
        base = (perm[torch.arange(n, device=dev) // 256] * 256 + torch.arange(n, device=dev) % 256).to(torch.int32)
        call = lambda i: ops.store_kvcache(key, value, kc[i % 2], vc[i % 2], base)
    elif a.case == "add_rmsnorm":
        xs, rs, nw = [rnd(16384, 4096) for _ in range(2)], [rnd(16384, 4096) for _ in range(2)], rnd(4096)
        call = lambda i: ops.add_rmsnorm(xs[i % 2], rs[i % 2], nw, 1e-6)
    elif a.case == "embed":
        w = rnd(151936, 4096)
        ids = [torch.randint(0, 151936, (16384,), device=dev, generator=g) for _ in range(2)]
        call = lambda i: ops.embed(ids[i % 2], w, 0, 151936, 1)
    else:
        raise SystemExit(f"unknown case {a.case}")
    with torch.inference_mode():
        for i in range(a.launches):
            call(i)
    torch.cuda.synchronize()
    shutdown_runtime()
    dist.destroy_process_group()
    print("done", a.case)


if __name__ == "__main__":
    main()
