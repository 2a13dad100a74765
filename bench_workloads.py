"""The two other BASELINE workloads, behind `bench.py --workload cfg2|cfg5` (same JSON line as the default workload).

cfg2  the reference's own bench.py workload (bench.py:9-27): Qwen3-0.6B random-init bf16 on one GPU, 256 sequences,
      prompt ids uniform in [0, 10000], prompt and output lengths uniform in [100, 1024], temperature 0.6, ignore_eos;
      total output tokens / wall time.  The batches are formed as the reference's scheduler forms them
      (nanovllm/engine/scheduler.py:25-58: whole prompts up to 16384 tokens per prefill step, then every running
      sequence decodes one token per step); tokens come from the LM head fused with the sampler.
cfg5  long-context prefill of Qwen3-32B random-init bf16 at tensor-parallel size 8: 4 sequences of 32768 uniform-random
      tokens in 16384-token chunks (nanovllm/engine/scheduler.py:42-48: only the first waiting sequence is chunked), KV
      blocks taken from a random permutation of the free list; prefill tokens / second.
"""
from __future__ import annotations

import json
import os
import random
import time


def _setup(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    entry.load_package()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torchrun"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29579")
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl" if world > 1 else "gloo", rank=rank, world_size=world)
    return torch, dist, rank, world, local


def _sync(torch, dist, world):
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()


def _max_over_ranks(torch, dist, world, v):
    if world == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_cfg5(args, peaks, clock_sampler_cls) -> None:
    torch, dist, rank, world, local = _setup(args)
    from nanovllm_b200.engine.model_runner import QWEN3_32B, ModelConfig, ModelRunner, Seq, sequential_block_tables
    n_seqs, seq_len, chunk, bs = 4, 32768, 16384, 256
    cfg = ModelConfig(**QWEN3_32B)
    blocks_per_seq = seq_len // bs
    runner = ModelRunner(cfg, max_num_seqs=n_seqs, max_model_len=seq_len, max_num_batched_tokens=chunk, num_kvcache_blocks=n_seqs * blocks_per_seq,
                         enforce_eager=True, oneshot_tokens=1024, seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab_size, (n_seqs, seq_len), generator=g).tolist()
    perm = list(range(n_seqs * blocks_per_seq))
    random.Random(0).shuffle(perm)  # the free list after some traffic: consecutive blocks of a sequence are scattered
    tables = sequential_block_tables([seq_len] * n_seqs, bs, permutation=perm)

    def one_pass():
        """All sequences from scratch: 8 steps of one 16384-token chunk each; returns the tokens sampled at the sequence ends."""
        out = []
        for p, bt in zip(prompts, tables):
            s = Seq(p, bt)
            for start in range(0, seq_len, chunk):
                s.num_cached_tokens = start
                toks = runner.step([s], True, num_new=[chunk])
            out.append(toks[0])
        return out

    K, W = max(1, min(args.steps, 4)), 1
    for _ in range(W):
        first = one_pass()
    _sync(torch, dist, world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with clock_sampler_cls(local) as clocks:
        e0.record()
        for _ in range(K):
            again = one_pass()
        e1.record()
        _sync(torch, dist, world)
    ms = _max_over_ranks(torch, dist, world, e0.elapsed_time(e1))
    runner.runtime.check_status()
    tokens = K * n_seqs * seq_len
    c = QWEN3_32B
    per_layer = c["hidden_size"] * (c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"] + c["num_attention_heads"] * c["head_dim"] * c["hidden_size"] \
        + 3 * c["hidden_size"] * c["intermediate_size"]
    gemm_flops = 2.0 * per_layer * c["num_hidden_layers"] * tokens
    attn_flops = 4.0 * c["num_attention_heads"] * c["head_dim"] * c["num_hidden_layers"] * K * n_seqs * (seq_len * (seq_len + 1) / 2)
    tf_per_gpu = (gemm_flops + attn_flops) / world / (ms * 1e-3) / 1e12
    if rank == 0:
        line = {"metric": "qwen3_32b_prefill_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"Qwen3-32B random-init bf16 long-context prefill, {n_seqs} x {seq_len} uniform-random tokens in {chunk}-token chunks, "
                                       f"paged KV (block 256) from a shuffled free list, TP={world}; one step = all {n_seqs} sequences",
                           "l2": "every chunk streams the rank's weight shard (8 GB at TP=8) and activations far larger than the 126 MB L2"},
                "clocks": clocks.summary(), "e2e": {"value": tokens / (ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": n_seqs * seq_len * 20,
                                                    "d2h_bytes_per_step": 8 * (seq_len // chunk) * n_seqs,
                                                    "note": "timed through ModelRunner.step(): token ids, positions and slot mapping copied from pinned host memory every chunk, sampled token read back"},
                "gpu_launches": None,
                "roofline": {"bound": "tensor", "achieved": tf_per_gpu, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": tf_per_gpu / peaks["bf16_tflops_sustained"],
                             "what": "GEMM + causal attention flops per GPU over the step time (whole step, all kernels and the attention library call)", "traffic": None},
                "parity": {"same_tokens_on_repeat": first == again}}
        from nanovllm_b200 import _abi
        line["gpu_launches"] = _abi.launch_count()
        print(json.dumps(line), flush=True)
    runner.exit()
    dist.destroy_process_group()


def run_cfg2(args, peaks, clock_sampler_cls) -> None:
    torch, dist, rank, world, local = _setup(args)
    from nanovllm_b200.engine.model_runner import QWEN3_0_6B, ModelConfig, ModelRunner, Seq, sequential_block_tables
    num_seqs, bs, max_batched = 256, 256, 16384
    random.seed(0)
    prompts = [[random.randint(0, 10000) for _ in range(random.randint(100, 1024))] for _ in range(num_seqs)]
    max_tokens = [random.randint(100, 1024) for _ in range(num_seqs)]
    tables = sequential_block_tables([len(p) + m for p, m in zip(prompts, max_tokens)], bs)
    runner = ModelRunner(ModelConfig(**QWEN3_0_6B), max_num_seqs=num_seqs, max_model_len=4096, max_num_batched_tokens=max_batched,
                         num_kvcache_blocks=sum(len(t) for t in tables), oneshot_tokens=1024, seed=0)

    def generate():
        """Prefill in batches of whole prompts (at most 16384 tokens), then decode every running sequence one token per
        step until each has produced its max_tokens (ignore_eos).  Returns (output tokens, decode steps)."""
        seqs = [Seq(list(p), bt) for p, bt in zip(prompts, tables)]
        left = list(max_tokens)
        i = 0
        while i < num_seqs:  # prefill
            j, n = i, 0
            while j < num_seqs and n + len(seqs[j]) <= max_batched:
                n += len(seqs[j])
                j += 1
            toks = runner.step(seqs[i:j], True, temperatures=[0.6] * (j - i))
            for k, t in zip(range(i, j), toks):
                seqs[k].token_ids.append(t)
                left[k] -= 1
            i = j
        running = [k for k in range(num_seqs) if left[k] > 0]
        steps = 0
        while running:
            toks = runner.step([seqs[k] for k in running], False, temperatures=[0.6] * len(running))
            for k, t in zip(running, toks):
                seqs[k].token_ids.append(t)
                left[k] -= 1
            running = [k for k in running if left[k] > 0]
            steps += 1
        return sum(max_tokens), steps

    runner.step([Seq([1, 2, 3, 4], [0])], True, temperatures=[1.0])  # the reference's warm-up request
    _sync(torch, dist, world)
    with clock_sampler_cls(local) as clocks:
        t0 = time.time()
        total, steps = generate()
        torch.cuda.synchronize()
        seconds = time.time() - t0
    runner.runtime.check_status()
    if rank == 0:
        from nanovllm_b200 import _abi
        line = {"metric": "qwen3_0_6b_bench_output_tokens_per_s", "value": total / seconds, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": 1,
                "ms_per_step": seconds * 1e3 / max(1, steps), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"the reference bench.py workload: Qwen3-0.6B random-init bf16, {num_seqs} sequences, prompt and output lengths uniform in [100, 1024], "
                                       f"temperature 0.6, ignore_eos, CUDA graphs, TP={world}; value = total output tokens / wall time (as the reference prints it)",
                           "l2": "decode steps stream the 1.2 GB of weights and the KV cache, far more than the 126 MB L2"},
                "clocks": clocks.summary(),
                "e2e": {"value": total / seconds, "unit": "tok/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                        "note": "wall clock through ModelRunner.step() with host batch state: this workload has no device-resident variant"},
                "gpu_launches": _abi.launch_count(), "total_output_tokens": total, "seconds": seconds}
        print(json.dumps(line), flush=True)
    runner.exit()
    dist.destroy_process_group()
