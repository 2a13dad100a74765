"""CPU timing of the reference's formulation of the path (TEST/BENCH INFRASTRUCTURE).

What is timed is the reference's own arithmetic for one decoder layer's
tensor-parallel path, written with the calls the reference makes:
F.linear for the qkv / gate_up projections (nanovllm/layers/linear.py:73),
F.linear + dist.all_reduce over gloo for o_proj / down_proj
(nanovllm/layers/linear.py:153-155), the eager add + RMSNorm
(nanovllm/layers/layernorm.py:28-40) and SiLU*mul
(nanovllm/layers/activation.py:8-11), in bf16 on the host cores.  Attention
itself (a library outside the path), the embedding and the LM head are left
out, which favours the CPU figure.  One process per tensor-parallel rank,
`cores // world` torch threads each.

Only bench.py (its cpu_baseline leg and its --impl reference arm) uses this.
"""
from __future__ import annotations

import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F


def _add_rms(x, residual, w, eps):
    s = x.float().add_(residual.float())
    new_res = s.to(x.dtype)
    var = s.pow(2).mean(dim=-1, keepdim=True)
    s.mul_(torch.rsqrt(var + eps))
    return s.to(x.dtype).mul_(w), new_res


def _layer_worker(rank, world, port, shape, m, threads, warmup, steps, max_seconds, q):
    torch.set_num_threads(max(1, threads))
    if world > 1:
        dist.init_process_group("gloo", f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    H, nq, nkv, hd, I = shape["hidden"], shape["n_heads"], shape["n_kv_heads"], shape["head_dim"], shape["intermediate"]
    g = torch.Generator().manual_seed(1234 + rank)
    bf = torch.bfloat16
    w_qkv = (torch.randn((nq + 2 * nkv) * hd // world, H, generator=g) * 0.02).to(bf)
    w_o = (torch.randn(H, nq * hd // world, generator=g) * 0.02).to(bf)
    w_gu = (torch.randn(2 * I // world, H, generator=g) * 0.02).to(bf)
    w_d = (torch.randn(H, I // world, generator=g) * 0.02).to(bf)
    n1 = torch.ones(H, dtype=bf)
    x = torch.randn(m, H, generator=g).to(bf)
    residual = torch.randn(m, H, generator=g).to(bf)

    def layer(h, res):
        qkv = F.linear(h, w_qkv)
        attn = qkv[:, : nq * hd // world].contiguous()  # stand-in for the attention output (same shape)
        y = F.linear(attn, w_o)
        if world > 1:
            dist.all_reduce(y)
        h, res = _add_rms(y, res, n1, 1e-6)
        gu = F.linear(h, w_gu)
        a, b = gu.chunk(2, -1)
        act = F.silu(a) * b
        y = F.linear(act, w_d)
        if world > 1:
            dist.all_reduce(y)
        return _add_rms(y, res, n1, 1e-6)

    with torch.inference_mode():
        for _ in range(warmup):
            layer(x, residual)
        if world > 1:
            dist.barrier()
        times = []
        t_start = time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            layer(x, residual)
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - t_start > max_seconds:
                break
    if world > 1:
        # every rank must run the same number of steps: agree on the minimum done
        n = torch.tensor([len(times)])
        dist.all_reduce(n, op=dist.ReduceOp.MIN)
        times = times[: int(n.item())]
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        q.put(times)


def time_decoder_layer(shape: dict, m: int, world: int, warmup: int, steps: int, max_seconds: float = 25.0, port: int = 29811) -> dict:
    """Seconds per decoder layer of the reference formulation on the host CPU."""
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    threads = max(1, cores // world)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_worker, args=(r, world, port, shape, m, threads, warmup, steps, max_seconds, q)) for r in range(world)]
    for p in procs:
        p.start()
    times = q.get(timeout=max_seconds * 4 + 300)
    for p in procs:
        p.join(120)
    times = sorted(times)
    mean = sum(times) / len(times)
    return {"seconds_per_layer": mean, "median_seconds_per_layer": times[len(times) // 2], "steps": len(times), "cores": threads * world, "threads_per_rank": threads}
