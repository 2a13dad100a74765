"""Runs the UNMODIFIED reference engine (the install under baseline/_ref) on the GPUs of this box and prints its
throughput as one JSON line: the reference's NCCL build beside which bench.py reports this repository's numbers.

    python baseline/reference_engine.py --tp N --workload decode8b [--steps K] [--warmup W]
    python baseline/reference_engine.py --tp 1 --workload bench06b

What runs is the reference's own code path end to end: LLMEngine.add_request / step (scheduler, block manager,
ModelRunner.run with its CUDA graphs, flash-attn, NCCL all_reduce / gather over the process group it creates, its
Sampler).  The harness only supplies what a checkpoint directory would:

  * a temporary model directory holding a Qwen3 config.json and a two-token stub tokenizer (the engine asks the
    tokenizer for nothing but the EOS id when prompts are token-id lists and ignore_eos is set);
  * seeded random N(0, 0.02) weights instead of safetensors: the reference's loader
    (nanovllm/utils/loader.py) finds no file and would leave torch.empty garbage, so ModelRunner's `load_model` name
    is pointed at an initialiser, in every rank's process, before the runner is built.  Nothing else is patched.

Engine construction follows nanovllm/engine/llm_engine.py:17-34 line for line (spawned ranks, events, rank 0 in this
process) because the spawned ranks must run the initialiser too; everything after construction is the engine's own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from random import randint, seed

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

MODELS = {
    "qwen3-8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                     num_hidden_layers=36, vocab_size=151936, tie_word_embeddings=False),
    "qwen3-0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072,
                       num_hidden_layers=28, vocab_size=151936, tie_word_embeddings=True),
    "qwen3-32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600,
                      num_hidden_layers=64, vocab_size=151936, tie_word_embeddings=False),
}


def write_model_dir(path: str, model: str) -> None:
    cfg = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1e6,
               attention_bias=False, hidden_act="silu", dtype="bfloat16", **MODELS[model])
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    from tokenizers import Tokenizer, models
    from transformers import PreTrainedTokenizerFast
    tok = Tokenizer(models.WordLevel({"<unk>": 0, "<eos>": 1}, unk_token="<unk>"))
    PreTrainedTokenizerFast(tokenizer_object=tok, eos_token="<eos>", unk_token="<unk>").save_pretrained(path)


def _random_init(model, path):
    """Stands in for nanovllm.utils.loader.load_model: seeded N(0, 0.02) weights made on the device, norm weights 1."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(1234 + torch.cuda.current_device())
    for name, p in model.named_parameters():
        if "norm" in name:
            p.data.fill_(1.0)
        else:
            p.data.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0, 0.02, generator=g))


def _scrub_launcher_environment() -> None:
    """A launcher's variables must not reach the engine's own process group (tcp://localhost:2333, one rank per process
    it spawns): with TORCHELASTIC_USE_AGENT_STORE set every rank would become a client of a store nobody hosts."""
    for k in list(os.environ):
        if k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK", "ROLE_WORLD_SIZE",
                 "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS") or k.startswith("TORCHELASTIC_"):
            del os.environ[k]


def _rank_entry(config, rank, event):
    """What the engine spawns for ranks > 0 (nanovllm/engine/llm_engine.py:26: target=ModelRunner), with the initialiser."""
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import nanovllm.engine.model_runner as mr
    mr.load_model = _random_init
    mr.ModelRunner(config, rank, event)


def build_engine(model_dir: str, **kwargs):
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import atexit
    from dataclasses import fields

    import torch.multiprocessing as mp
    from transformers import AutoTokenizer

    import nanovllm.engine.model_runner as mr
    from nanovllm.config import Config
    from nanovllm.engine.llm_engine import LLMEngine
    from nanovllm.engine.scheduler import Scheduler
    from nanovllm.engine.sequence import Sequence
    mr.load_model = _random_init

    class Engine(LLMEngine):
        def __init__(self, model, **kw):  # nanovllm/engine/llm_engine.py:17-34 with _rank_entry as the spawn target
            config_fields = {f.name for f in fields(Config)}
            config = Config(model, **{k: v for k, v in kw.items() if k in config_fields})
            Sequence.block_size = config.kvcache_block_size
            self.ps, self.events = [], []
            ctx = mp.get_context("spawn")
            for i in range(1, config.tensor_parallel_size):
                event = ctx.Event()
                process = ctx.Process(target=_rank_entry, args=(config, i, event))
                process.start()
                self.ps.append(process)
                self.events.append(event)
            self.model_runner = mr.ModelRunner(config, 0, self.events)
            self.tokenizer = AutoTokenizer.from_pretrained(config.model, use_fast=True)
            config.eos = self.tokenizer.eos_token_id
            self.scheduler = Scheduler(config)
            atexit.register(self.exit)

    return Engine(model_dir, **kwargs)


def run_decode(engine, batch: int, prompt_len: int, steps: int, warmup: int, vocab: int) -> dict:
    """Config "Qwen3-8B decode": `batch` prompts of `prompt_len` uniform-random ids, greedy (the reference's sampler at
    temperature 1e-6), ignore_eos; decode steps timed one by one around engine.step() (the reference's own per-step
    clock, nanovllm/engine/llm_engine.py:72-79), the first `warmup` decode steps left out."""
    import torch
    from nanovllm.sampling_params import SamplingParams
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, vocab, (batch, prompt_len), generator=g).tolist()
    sp = SamplingParams(temperature=1e-6, ignore_eos=True, max_tokens=steps + warmup + 1)
    for p in prompts:
        engine.add_request(p, sp)
    decode_times, prefill_tokens, prefill_s = [], 0, 0.0
    while not engine.is_finished() and len(decode_times) < steps + warmup:
        t0 = time.perf_counter()
        _, num_tokens = engine.step()
        dt = time.perf_counter() - t0
        if num_tokens > 0:
            prefill_tokens += num_tokens
            prefill_s += dt
        else:
            assert -num_tokens == batch, "the scheduler did not decode the whole batch in one step"
            decode_times.append(dt)
    timed = decode_times[warmup:]
    total = sum(timed)
    return {"value": batch * len(timed) / total, "unit": "tok/s", "steps": len(timed), "warmup": warmup, "ms_per_step": total / len(timed) * 1e3,
            "prefill_tok_s": prefill_tokens / prefill_s if prefill_s else None}


def run_bench06b(engine, num_seqs: int = 256) -> dict:
    """The reference's own bench.py workload (bench.py:9-27): 256 sequences, prompt ids uniform in [0, 10000], prompt
    and output lengths uniform in [100, 1024], temperature 0.6, ignore_eos; total output tokens / wall time."""
    from nanovllm.sampling_params import SamplingParams
    seed(0)
    prompts = [[randint(0, 10000) for _ in range(randint(100, 1024))] for _ in range(num_seqs)]
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_tokens=randint(100, 1024)) for _ in range(num_seqs)]
    engine.generate([[1, 2, 3, 4]], SamplingParams(max_tokens=8), use_tqdm=False)  # the reference's warm-up request
    t0 = time.time()
    engine.generate(prompts, sps, use_tqdm=False)
    t = time.time() - t0
    total = sum(sp.max_tokens for sp in sps)
    return {"value": total / t, "unit": "tok/s", "total_output_tokens": total, "seconds": t, "num_seqs": num_seqs}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--workload", default="decode8b", choices=["decode8b", "bench06b"])
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--num-seqs", type=int, default=256)
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(REF, "nanovllm")):
        print(json.dumps({"impl": "reference-engine", "unavailable": "the reference is not installed under baseline/_ref (python baseline/install_reference.py)"}))
        return
    _scrub_launcher_environment()
    model = "qwen3-8b" if a.workload == "decode8b" else "qwen3-0.6b"
    with tempfile.TemporaryDirectory() as d:
        write_model_dir(d, model)
        if a.workload == "decode8b":
            engine = build_engine(d, tensor_parallel_size=a.tp, max_num_seqs=a.batch, max_model_len=4096, enforce_eager=False)
            res = run_decode(engine, a.batch, a.prompt_len, a.steps, a.warmup, MODELS[model]["vocab_size"])
            res["config"] = f"Qwen3-8B random-init bf16 decode, batch {a.batch}, {a.prompt_len}-token prompts, greedy, CUDA graphs, TP={a.tp}"
        else:
            engine = build_engine(d, tensor_parallel_size=a.tp, max_model_len=4096, enforce_eager=False)
            res = run_bench06b(engine, a.num_seqs)
            res["config"] = f"Qwen3-0.6B random-init bf16, the reference bench.py workload ({a.num_seqs} sequences, temperature 0.6), TP={a.tp}"
        res.update({"impl": "reference-engine", "tp": a.tp, "what": "unmodified reference LLMEngine (NCCL, flash-attn, CUDA graphs), random-init weights"})
        print(json.dumps(res), flush=True)
        engine.exit()
        import atexit
        atexit.unregister(engine.exit)


if __name__ == "__main__":
    main()
