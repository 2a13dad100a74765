"""CPU timing of the reference's tensor-parallel layer path (TEST/BENCH INFRASTRUCTURE).

What is timed is one decoder layer's tensor-parallel path on the host cores, in
bf16, one process per tensor-parallel rank over gloo, `cores // world` torch
threads each:

  kind "reference"  the reference's own modules, imported from its install
                    under baseline/_ref: QKVParallelLinear,
                    RowParallelLinear (F.linear + dist.all_reduce,
                    nanovllm/layers/linear.py:153-155), RMSNorm
                    (nanovllm/layers/layernorm.py:28-40, run eagerly),
                    MergedColumnParallelLinear and SiluAndMul
                    (nanovllm/layers/activation.py:8-11), called in the order
                    nanovllm/models/qwen3.py:146-159 calls them.
  kind "port"       the same arithmetic restated with plain torch calls, used
                    only when the install is absent.

Attention itself (a GPU library outside the path), the embedding and the LM
head are left out, which favours the CPU figure.

Only bench.py (its cpu_baseline leg and its --impl reference arm) and the
tests use this.
"""
from __future__ import annotations

import contextlib
import datetime
import os
import queue as queue_mod
import socket
import sys
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_INSTALL = os.path.join(ROOT, "baseline", "_ref")

# Variables a launcher (torch.distributed.run) sets for ITS ranks.  The gloo ranks started here form their own
# group; with TORCHELASTIC_USE_AGENT_STORE inherited every one of them would become a client of a store that
# nobody hosts.
_LAUNCHER_VARS = ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE",
                  "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS", "MKL_NUM_THREADS")


def reference_available() -> bool:
    return os.path.isdir(os.path.join(REF_INSTALL, "nanovllm"))


@contextlib.contextmanager
def _child_environment():
    """The environment the spawned ranks inherit: no launcher variables, dynamo off (the reference decorates
    its elementwise functions with torch.compile; inductor has no working CPU toolchain here)."""
    saved = dict(os.environ)
    try:
        for k in list(os.environ):
            if k in _LAUNCHER_VARS or k.startswith("TORCHELASTIC_") or k.startswith("TORCH_NCCL_") or k.startswith("NCCL_"):
                del os.environ[k]
        os.environ["TORCHDYNAMO_DISABLE"] = "1"
        os.environ["CUDA_VISIBLE_DEVICES"] = ""
        yield
    finally:
        os.environ.clear()
        os.environ.update(saved)


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _add_rms(x, residual, w, eps):
    s = x.float().add_(residual.float())
    new_res = s.to(x.dtype)
    var = s.pow(2).mean(dim=-1, keepdim=True)
    s.mul_(torch.rsqrt(var + eps))
    return s.to(x.dtype).mul_(w), new_res


def _build_port_layer(shape, world, g):
    H, nq, nkv, hd, I = shape["hidden"], shape["n_heads"], shape["n_kv_heads"], shape["head_dim"], shape["intermediate"]
    bf = torch.bfloat16
    w_qkv = (torch.randn((nq + 2 * nkv) * hd // world, H, generator=g) * 0.02).to(bf)
    w_o = (torch.randn(H, nq * hd // world, generator=g) * 0.02).to(bf)
    w_gu = (torch.randn(2 * I // world, H, generator=g) * 0.02).to(bf)
    w_d = (torch.randn(H, I // world, generator=g) * 0.02).to(bf)
    n1 = torch.ones(H, dtype=bf)
    q_cols = nq * hd // world

    def layer(h, res):
        qkv = F.linear(h, w_qkv)
        attn = qkv[:, :q_cols].contiguous()  # stand-in for the attention output (same shape)
        y = F.linear(attn, w_o)
        if world > 1:
            dist.all_reduce(y)
        h, res = _add_rms(y, res, n1, 1e-6)
        gu = F.linear(h, w_gu)
        a, b = gu.chunk(2, -1)
        y = F.linear(F.silu(a) * b, w_d)
        if world > 1:
            dist.all_reduce(y)
        return _add_rms(y, res, n1, 1e-6)

    return layer


def _build_reference_layer(shape, world, g):
    """One decoder layer's tensor-parallel modules, the reference's own classes (they read rank and world from
    the default process group, nanovllm/layers/linear.py:23-24)."""
    if REF_INSTALL not in sys.path:
        sys.path.insert(0, REF_INSTALL)
    from nanovllm.layers.activation import SiluAndMul
    from nanovllm.layers.layernorm import RMSNorm
    from nanovllm.layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
    H, nq, nkv, hd, I = shape["hidden"], shape["n_heads"], shape["n_kv_heads"], shape["head_dim"], shape["intermediate"]
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        qkv_proj = QKVParallelLinear(H, hd, nq, nkv, bias=False)
        o_proj = RowParallelLinear(nq * hd, H, bias=False)
        gate_up = MergedColumnParallelLinear(H, [I, I], bias=False)
        down = RowParallelLinear(I, H, bias=False)
        post_norm, next_norm, act = RMSNorm(H, eps=1e-6), RMSNorm(H, eps=1e-6), SiluAndMul()
    finally:
        torch.set_default_dtype(prev)
    for lin in (qkv_proj, o_proj, gate_up, down):
        lin.weight.data.copy_(torch.randn(lin.weight.shape, generator=g) * 0.02)
    q_cols = nq * hd // world

    def layer(h, res):
        qkv = qkv_proj(h)
        attn = qkv[:, :q_cols].contiguous()  # stand-in for the attention output (same shape)
        h, res = post_norm(o_proj(attn), res)
        return next_norm(down(act(gate_up(h))), res)

    return layer


def _layer_worker(rank, world, port, shape, m, threads, warmup, steps, max_seconds, kind, q):
    try:
        torch.set_num_threads(max(1, threads))
        if world > 1 or kind == "reference":  # the reference's layers need a default group even at world size 1
            store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=60))
            dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
        g = torch.Generator().manual_seed(1234 + rank)
        layer = _build_reference_layer(shape, world, g) if kind == "reference" else _build_port_layer(shape, world, g)
        H = shape["hidden"]
        x = torch.randn(m, H, generator=g).to(torch.bfloat16)
        residual = torch.randn(m, H, generator=g).to(torch.bfloat16)
        with torch.inference_mode():
            for _ in range(max(1, warmup)):
                layer(x.clone(), residual.clone())
            # every rank runs the same number of timed passes, fixed before the loop from the slowest rank's pace
            t0 = time.perf_counter()
            layer(x.clone(), residual.clone())
            pace = torch.tensor([time.perf_counter() - t0], dtype=torch.float64)
            if world > 1:
                dist.all_reduce(pace, op=dist.ReduceOp.MAX)
            n = int(max(1, min(steps, max_seconds / max(pace.item(), 1e-6))))
            if world > 1:
                dist.barrier()
            times = []
            for _ in range(n):
                t0 = time.perf_counter()
                layer(x.clone(), residual.clone())
                times.append(time.perf_counter() - t0)
        if dist.is_initialized():
            if world > 1:
                dist.barrier()
            dist.destroy_process_group()
        if rank == 0:
            q.put(("ok", times))
    except Exception as ex:  # the parent must not wait for a rank that has died
        q.put(("error", f"rank {rank}: {ex!r}"))
        raise


def time_decoder_layer(shape: dict, m: int, world: int, warmup: int, steps: int, max_seconds: float = 25.0, kind: str | None = None) -> dict:
    """Seconds per decoder layer of the reference's path on the host CPU (see the module docstring)."""
    if kind is None:
        kind = "reference" if reference_available() else "port"
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    threads = max(1, cores // world)
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with _child_environment():
        procs = [ctx.Process(target=_layer_worker, args=(r, world, port, shape, m, threads, warmup, steps, max_seconds, kind, q)) for r in range(world)]
        for p in procs:
            p.start()
    deadline = time.monotonic() + 2 * max_seconds + 180  # start-up (imports, rendezvous) + warm-up + the timed passes
    result = None
    try:
        while result is None:
            try:
                result = q.get(timeout=1.0)
            except queue_mod.Empty:
                dead = [p for p in procs if p.exitcode not in (None, 0)]
                if dead:
                    raise RuntimeError(f"a CPU baseline rank exited with code {dead[0].exitcode}")
                if time.monotonic() > deadline:
                    raise TimeoutError("the CPU baseline ranks did not finish in time")
        if result[0] != "ok":
            raise RuntimeError(result[1])
    finally:
        for p in procs:
            p.join(5 if result is None else 60)
            if p.is_alive():
                p.terminate()
    times = sorted(result[1])
    mean = sum(times) / len(times)
    return {"seconds_per_layer": mean, "median_seconds_per_layer": times[len(times) // 2], "steps": len(times), "cores": threads * world,
            "threads_per_rank": threads, "kind": kind}
