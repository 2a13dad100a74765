"""A small random-init Qwen3 through the model runner (prefill, eager decode,
CUDA-graph decode) against the CPU oracle of the whole model, one B200."""
import pytest
import torch

from oracle import tp_path as O
from tests.gpu_util import ensure_group

pytestmark = pytest.mark.gpu

SHAPE = O.QwenShape(hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, intermediate=512, n_layers=3, vocab=2048)


def _attention_backend():
    """The attention library is outside the path; use it when it runs on this GPU."""
    from nanovllm_b200.layers.attention import Attention
    try:
        from flash_attn import flash_attn_with_kvcache
        q = torch.zeros(1, 1, 2, 128, device="cuda", dtype=torch.bfloat16)
        kc = torch.zeros(1, 256, 1, 128, device="cuda", dtype=torch.bfloat16)
        flash_attn_with_kvcache(q, kc, kc, cache_seqlens=torch.ones(1, dtype=torch.int32, device="cuda"),
                                block_table=torch.zeros(1, 1, dtype=torch.int32, device="cuda"), causal=True)
        torch.cuda.synchronize()
        Attention.backend = "flash_attn"
    except Exception:
        Attention.backend = "sdpa"
    return Attention.backend


@pytest.mark.parametrize("enforce_eager", [True, False])
def test_small_qwen3_matches_oracle(pkg, enforce_eager):
    ensure_group()
    from nanovllm_b200.engine.model_runner import ModelConfig, ModelRunner, Seq, sequential_block_tables
    _attention_backend()
    weights = O.init_full_weights(SHAPE, seed=17)
    cfg = ModelConfig(hidden_size=SHAPE.hidden, num_attention_heads=SHAPE.n_heads, num_key_value_heads=SHAPE.n_kv_heads, head_dim=SHAPE.head_dim,
                      intermediate_size=SHAPE.intermediate, num_hidden_layers=SHAPE.n_layers, vocab_size=SHAPE.vocab,
                      max_position_embeddings=1024)
    runner = ModelRunner(cfg, max_num_seqs=16, max_model_len=1024, max_num_batched_tokens=2048, num_kvcache_blocks=16,
                         enforce_eager=enforce_eager, oneshot_tokens=256, full_weights=weights)
    try:
        g = torch.Generator().manual_seed(3)
        lens = [37, 300, 5]
        seqs = [Seq(torch.randint(0, SHAPE.vocab, (n,), generator=g).tolist()) for n in lens]
        for s, bt in zip(seqs, sequential_block_tables([n + 8 for n in lens], 256)):
            s.block_table = bt
        oracle = O.QwenOracle(SHAPE, weights, world=1, max_pos=1024)

        def oracle_step(new_tokens):
            ids = torch.tensor([t for ts in new_tokens for t in ts])
            pos = torch.cat([torch.arange(len(s) - len(ts), len(s)) for s, ts in zip(seqs, new_tokens)])
            return oracle.forward(ids, pos, list(range(len(seqs))), [len(ts) for ts in new_tokens]).float()

        agree = total = 0
        # prefill, then 6 teacher-forced decode steps (the oracle's token is fed to both sides)
        ref_logits = oracle_step([s.token_ids for s in seqs])
        ids, pos = runner.prepare_prefill(seqs)
        logits = runner.run_model(ids, pos, True).float().cpu()
        for step in range(7):
            err = (logits - ref_logits).abs().max().item()
            scale = ref_logits.abs().max().item()
            assert err <= 2e-2 + 3e-2 * scale, f"step {step}: logits differ by {err} (scale {scale})"
            top2 = ref_logits.topk(2, dim=-1).values
            decided = (top2[:, 0] - top2[:, 1]) > 2 * err
            agree += (logits.argmax(-1) == ref_logits.argmax(-1))[decided].sum().item()
            total += decided.sum().item()
            nxt = ref_logits.argmax(-1).tolist()
            for s, t in zip(seqs, nxt):
                s.token_ids.append(t)
            if step == 6:
                break
            ref_logits = oracle_step([[t] for t in nxt])
            ids, pos = runner.prepare_decode(seqs)
            logits = runner.run_model(ids, pos, False).float().cpu()
        runner.runtime.check_status()
        assert total > 0 and agree == total, f"greedy tokens agree on {agree}/{total} decided positions"
    finally:
        runner.exit()


def test_step_returns_greedy_tokens(pkg):
    ensure_group()
    from nanovllm_b200.engine.model_runner import ModelConfig, ModelRunner, Seq, sequential_block_tables
    _attention_backend()
    cfg = ModelConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=512,
                      num_hidden_layers=2, vocab_size=2048, max_position_embeddings=1024)
    runner = ModelRunner(cfg, max_num_seqs=8, max_model_len=512, max_num_batched_tokens=1024, num_kvcache_blocks=8, oneshot_tokens=128, seed=1)
    try:
        seqs = [Seq(list(range(10, 10 + n))) for n in (12, 200)]
        for s, bt in zip(seqs, sequential_block_tables([256, 256], 256)):
            s.block_table = bt
        toks = runner.step(seqs, True)
        assert len(toks) == 2 and all(0 <= t < 2048 for t in toks)
        for _ in range(3):
            for s, t in zip(seqs, toks):
                s.token_ids.append(t)
            toks = runner.step(seqs, False)
        sampled = runner.step([Seq(s.token_ids + [t], s.block_table) for s, t in zip(seqs, toks)], False, temperatures=[0.6, 0.6])
        assert len(sampled) == 2
    finally:
        runner.exit()
