"""Benchmark of the tensor-parallel layer path: Qwen3-8B decode tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N > 1 is launched as one process per GPU (torchrun); rank/world come from the
environment.  Workload: Qwen3-8B, random-init bf16 weights, 64 sequences with
1024-token uniform-random prompts (prefilled through the same kernels, not
timed), then K greedy decode steps of the whole batch at tensor-parallel size
N.  One step = one new token for each of the 64 sequences.

Prints one JSON line (rank 0).  `value`: decode tokens/s with the batch state
resident on the device (one CUDA graph per step: model, LM head + gather,
greedy pick, token broadcast, next inputs).  `e2e`: the same through the
runner's public step() with host-side batch state: pinned host->device copies
of the step's inputs and a device->host read of the chosen tokens every step.

--impl reference: the reference's own formulation of the layer path (F.linear
+ gloo all_reduce + eager RMSNorm, oracle/cpu_baseline.py) timed on the host
cores; rank 0 alone runs it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "qwen3_8b_decode_tokens_per_s"
BATCH, PROMPT_LEN = 64, 1024
SHAPE_8B = dict(hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, intermediate=12288, n_layers=36, vocab=151936)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
def ncu_traffic_bytes(tp: int):
    """DRAM bytes per launch of the kernel the roofline leg times, from the ncu capture on record for this tensor-parallel
    size (a small JSON beside the capture summaries); None where no capture exists."""
    try:
        table = json.load(open(os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")))
        entry = table.get(f"gate_up_silu_mul_m{BATCH}_n{2 * SHAPE_8B['intermediate'] // tp}_k{SHAPE_8B['hidden']}_tp{tp}")
        return entry["bytes"] if entry else None
    except Exception:
        return None


def workload(tp: int) -> dict:
    return {"workload": f"Qwen3-8B random-init bf16 decode, batch {BATCH}, {PROMPT_LEN}-token uniform-random prompts, greedy, CUDA graphs, TP={tp}",
            "batch": BATCH, "prompt_len": PROMPT_LEN, "tp": tp, "kv_block": 256,
            "l2": "no flush needed: every step streams the rank's whole weight shard (16.4 GB / TP) and the KV cache, far more than the 126 MB L2"}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return json.load(open(path)), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_reference(world: int, warmup: int, steps: int, max_seconds: float) -> dict:
    """tokens/s of the reference's layer path on the host CPU: 64 tokens per
    decode step, 36 decoder layers per step, one decoder layer per sample."""
    from oracle import cpu_baseline
    r = cpu_baseline.time_decoder_layer(SHAPE_8B, BATCH, world, warmup, steps, max_seconds)
    step_s = r["seconds_per_layer"] * SHAPE_8B["n_layers"]
    what = ("the reference's own QKVParallelLinear, RowParallelLinear (F.linear + gloo all_reduce), RMSNorm, MergedColumnParallelLinear and SiluAndMul "
            "modules" if r["kind"] == "reference" else "a restatement of the reference's modules (F.linear + gloo all_reduce + eager RMSNorm)")
    return {"value": BATCH / step_s, "unit": "tok/s", "cores": r["cores"], "kind": r["kind"],
            "sample": f"{r['steps']} timed passes of ONE decoder layer's tensor-parallel path (qkv, o_proj+all_reduce+add-RMSNorm, gate_up, SiLU*mul, "
                      f"down_proj+all_reduce+add-RMSNorm) through {what} at M={BATCH}, bf16, {world} gloo rank(s) x {r['threads_per_rank']} threads; "
                      "scaled by 36 layers; attention, embedding and LM head left out",
            "ms_per_step": step_s * 1e3, "steps": r["steps"]}


def run_reference(args) -> None:
    """The reference arm: rank 0 alone times the CPU path (it starts its own gloo ranks); under a launcher the
    other ranks have nothing to do."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tp = args.gpus
    steps = max(1, args.steps)
    warmup = max(1, min(args.warmup, 3))
    ref = cpu_reference(tp, warmup, steps, max_seconds=60.0)
    line = {"metric": METRIC, "value": ref["value"], "unit": "tok/s", "n_gpus": tp, "steps": ref["steps"], "warmup": warmup,
            "ms_per_step": ref["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload(tp), "impl": "reference",
            "cpu_baseline": {k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": ref["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def reference_engine_gpu(tp: int, steps: int, warmup: int, timeout_s: float = 600.0) -> dict:
    """The unmodified reference engine (NCCL, flash-attn, CUDA graphs) on the same GPUs and workload, in a process
    group of its own (baseline/reference_engine.py); returns its JSON line, or why there is none."""
    import signal
    script = os.path.join(ROOT, "baseline", "reference_engine.py")
    cmd = [sys.executable, script, "--tp", str(tp), "--workload", "decode8b", "--steps", str(steps), "--warmup", str(warmup),
           "--batch", str(BATCH), "--prompt-len", str(PROMPT_LEN)]
    env = {k: v for k, v in os.environ.items() if not (k.startswith("TORCHELASTIC_") or k in (
        "RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE", "ROLE_NAME",
        "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS"))}
    try:
        proc = subprocess.Popen(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
        try:
            out, err = proc.communicate(timeout=timeout_s)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)  # the engine's own process group: rank 0 and the ranks it spawned
            proc.communicate()
            return {"unavailable": f"the reference engine did not finish within {timeout_s:.0f} s"}
        lines = [l for l in out.splitlines() if l.startswith("{")]
        if proc.returncode != 0 or not lines:
            return {"unavailable": f"the reference engine exited with code {proc.returncode}: {(err or out)[-300:]}"}
        return json.loads(lines[-1])
    except Exception as ex:
        return {"unavailable": repr(ex)[:300]}


def run_b200(args) -> None:
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    entry.load_package()
    from nanovllm_b200 import _abi, ops
    from nanovllm_b200.engine.model_runner import QWEN3_8B, ModelConfig, ModelRunner, ResidentDecoder, Seq, sequential_block_tables

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torchrun"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl" if world > 1 else "gloo", rank=rank, world_size=world)
    dev = torch.device("cuda", local)
    K, W = args.steps, max(3, args.warmup)
    max_len = ((PROMPT_LEN + K + W + 8 + 255) // 256) * 256
    blocks_per_seq = max_len // 256
    runner = ModelRunner(ModelConfig(**QWEN3_8B), max_num_seqs=BATCH, max_model_len=max_len, max_num_batched_tokens=16384,
                         num_kvcache_blocks=BATCH * blocks_per_seq, oneshot_tokens=1024, seed=0)
    resident = ResidentDecoder(runner, BATCH)

    # ---- prompts and prefill (not timed): 4 steps of 16 sequences, as the reference's scheduler would batch them
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, SHAPE_8B["vocab"], (BATCH, PROMPT_LEN), generator=g).tolist()
    tables = sequential_block_tables([max_len] * BATCH, 256)
    first = []
    for i in range(0, BATCH, 16):
        first += runner.step([Seq(list(p), bt) for p, bt in zip(prompts[i:i + 16], tables[i:i + 16])], True)

    def fresh_seqs():
        return [Seq(list(p) + [t], bt) for p, t, bt in zip(prompts, first, tables)]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident decode: `value` ----
    resident.load(fresh_seqs())
    for _ in range(W):
        resident.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        torch.cuda.nvtx.range_push("timed")
        e0.record()
        for _ in range(K):
            resident.replay()
        e1.record()
        barrier()
        torch.cuda.nvtx.range_pop()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    runner.runtime.check_status()
    launches = K * resident.kernels_per_step
    final_tokens = resident.tokens.tolist()
    assert all(0 <= t < SHAPE_8B["vocab"] for t in final_tokens)

    # ---- end to end through runner.step(): host batch state, H2D inputs + D2H tokens every step ----
    seqs = fresh_seqs()
    def e2e_step():
        toks = runner.step(seqs, False)
        for s, t in zip(seqs, toks):
            s.token_ids.append(t)
    for _ in range(W):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(K):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    h2d = BATCH * (8 + 8 + 4 + 4) + BATCH * blocks_per_seq * 4
    d2h = BATCH * 8

    # ---- roofline of the dominant kernel: the gate_up GEMM (largest share of the step), timed alone ----
    pk, pk_kind = peaks()
    layers = runner.model.model.layers
    x = torch.randn(BATCH, SHAPE_8B["hidden"], device=dev).bfloat16()
    n_local = 2 * SHAPE_8B["intermediate"] // world
    paired = [l.mlp.gate_up_proj.paired_weight() for l in layers]  # what the decoder layer launches: gate_up with SiLU*mul in the epilogue
    # one CUDA graph holds one launch per layer's weight (36 x 201 MB / TP: never L2-resident), so the host is out of the loop
    from nanovllm_b200.rowpar_microbench import time_in_graph
    with torch.inference_mode():
        k_us = time_in_graph(lambda i: ops.gemm_silu_mul(x, paired[i % len(layers)]), len(layers), 6 * len(layers))
    alg_bytes = 2.0 * (BATCH * SHAPE_8B["hidden"] + n_local * SHAPE_8B["hidden"] + BATCH * n_local // 2)
    achieved = alg_bytes / (k_us * 1e-6) / 1e9
    roofline = {"bound": "hbm", "kernel": f"{'gemm_kernel<64,SWAP,STORE> (stream-K)' if n_local // 128 > 148 else 'gemm_cluster_kernel<64,STORE>'} gate_up_proj + SiLU*mul, M={BATCH} N={n_local} K={SHAPE_8B['hidden']}", "achieved": achieved,
                "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "peak_kind": pk_kind + " (burst copy bandwidth)",
                "us_per_launch": k_us, "algorithmic_bytes": alg_bytes, "traffic": ncu_traffic_bytes(world)}
    # the whole step against the HBM bound: weights of the rank + KV read at the mean context length
    c = SHAPE_8B
    w_bytes = 2.0 * (c["n_layers"] * (c["hidden"] * (c["n_heads"] + 2 * c["n_kv_heads"]) * c["head_dim"] + c["hidden"] * c["n_heads"] * c["head_dim"]
                                      + 3 * c["hidden"] * c["intermediate"]) + c["vocab"] * c["hidden"]) / world
    kv_bytes = 2.0 * 2 * c["n_layers"] * BATCH * (PROMPT_LEN + W + K / 2) * c["n_kv_heads"] * c["head_dim"] / world
    step_ms = total_ms / K
    step_roof = {"bound": "hbm", "achieved": (w_bytes + kv_bytes) / (step_ms * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                 "frac": (w_bytes + kv_bytes) / (step_ms * 1e-3) / 1e9 / pk["hbm_gbs"], "bytes_per_step": w_bytes + kv_bytes}

    # ---- the fused row-parallel block next to F.linear + NCCL all_reduce + RMSNorm (N > 1) ----
    block_cmp = None
    if world > 1 and not args.skip_nccl:
        try:
            from nanovllm_b200 import rowpar_microbench as mb
            block_cmp = mb.compare_blocks([("o_proj", BATCH, c["hidden"], c["n_heads"] * c["head_dim"] // world),
                                           ("down_proj", BATCH, c["hidden"], c["intermediate"] // world)], pk, iters=200)
        except Exception as ex:  # the comparison is informative only
            block_cmp = {"error": repr(ex)[:200]}

    # ---- the whole model forward next to the reference's formulation of it (cuBLAS + NCCL + compiled elementwise) ----
    forward_cmp = None
    if args.forward_compare:
        try:
            from nanovllm_b200 import rowpar_microbench as mb
            resident.load(fresh_seqs())
            forward_cmp = mb.compare_model_forward(runner, BATCH)
        except Exception as ex:
            forward_cmp = {"error": repr(ex)[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        ref = cpu_reference(1, 1, 64, max_seconds=15.0)
        cpu = {k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")}

    # ---- parity of what was timed: the device-resident loop and step() must pick the same tokens ----
    resident.load(fresh_seqs())
    from_resident = []
    for _ in range(8):
        resident.replay()
        from_resident.append(resident.tokens.tolist())
    seqs = fresh_seqs()
    same = total = 0
    for k in range(8):
        toks = runner.step(seqs, False)
        for s_, t in zip(seqs, toks):
            s_.token_ids.append(t)
        same += sum(int(a == b) for a, b in zip(from_resident[k], toks))
        total += len(toks)
    runner.runtime.check_status()
    parity = {"resident_loop_vs_step_tokens_identical": f"{same}/{total}",
              "note": "greedy tokens of 8 decode steps of the 64 sequences through both timed paths; tests/test_gpu_decode_paths.py checks both against the oracle"}
    if block_cmp is not None and "error" not in block_cmp:
        parity["rowpar_block_within_bf16_tolerance_of_fp32"] = all(r.get("parity_vs_fp32", {}).get("within_tolerance", False) for r in block_cmp.values())

    clock_summary = clocks.summary()
    runner.exit()
    del resident, runner, layers, paired
    import gc
    gc.collect()
    torch.cuda.empty_cache()

    # ---- the unmodified reference engine (its NCCL build) on the same GPUs, after this arm has released them ----
    ref_gpu = None
    if not args.skip_reference_gpu:
        barrier()
        if rank == 0:
            ref_gpu = reference_engine_gpu(world, min(K, 64), 8)
        if world > 1:
            dist.barrier()

    if rank == 0:
        line = {"metric": METRIC, "value": BATCH * K / (total_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": workload(world), "clocks": clock_summary,
                "e2e": {"value": BATCH * K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / K},
                "gpu_launches": launches, "roofline": roofline, "step_roofline": step_roof, "cpu_baseline": cpu, "parity": parity}
        if block_cmp is not None:
            line["rowpar_block_us"] = block_cmp
        if forward_cmp is not None:
            line["model_forward_us"] = forward_cmp
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
            if "value" in ref_gpu:
                line["reference_gpu"]["b200_over_reference_e2e"] = line["e2e"]["value"] / ref_gpu["value"]
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg")
    ap.add_argument("--skip-nccl", action="store_true", help="omit the NCCL comparison of the row-parallel block")
    ap.add_argument("--forward-compare", action="store_true", help="also time a restatement of the reference's decode forward (cuBLAS + NCCL + "
                    "compiled elementwise) on the runner's weights; superseded by the run of the reference engine itself")
    ap.add_argument("--skip-reference-gpu", action="store_true", help="omit the run of the unmodified reference engine on the GPUs")
    ap.add_argument("--workload", default="decode8b", choices=["decode8b", "cfg2", "cfg5"],
                    help="decode8b: Qwen3-8B decode (the headline metric); cfg2: the reference bench.py workload (Qwen3-0.6B); cfg5: Qwen3-32B long prefill")
    args = ap.parse_args()
    if args.workload != "decode8b" and args.impl == "b200":
        import bench_workloads
        pk, _ = peaks()
        (bench_workloads.run_cfg2 if args.workload == "cfg2" else bench_workloads.run_cfg5)(args, pk, ClockSampler)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
