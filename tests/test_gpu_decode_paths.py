"""The decode paths the benchmark times, against each other and against the CPU oracle (one B200):

* ResidentDecoder.load() + K x replay()  (device-resident loop: what bench.py's `value` is timed on)
* K x ModelRunner.step()                 (host batch state, graph replay through _decode_graph_step: bench.py's `e2e`)
* the whole-model oracle, teacher-forced on the tokens the device produced

and chunked prefill (prepare_prefill(..., num_new=...) with a cached prefix, the reference's
nanovllm/engine/model_runner.py:129-170 with num_scheduled_tokens < len(seq)) against the oracle's logits.
"""
import pytest
import torch

from oracle import tp_path as O
from tests.gpu_util import ensure_group
from tests.test_gpu_model import _attention_backend

pytestmark = pytest.mark.gpu

SHAPE = O.QwenShape(hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, intermediate=512, n_layers=3, vocab=2048)


def _config(shape, max_pos=2048):
    from nanovllm_b200.engine.model_runner import ModelConfig
    return ModelConfig(hidden_size=shape.hidden, num_attention_heads=shape.n_heads, num_key_value_heads=shape.n_kv_heads, head_dim=shape.head_dim,
                       intermediate_size=shape.intermediate, num_hidden_layers=shape.n_layers, vocab_size=shape.vocab,
                       max_position_embeddings=max_pos, tie_word_embeddings=shape.tie)


def oracle_agreement(oracle, prompts, produced):
    """Teacher-forced: the oracle reads the tokens the device produced and, at every position, names its own greedy
    token.  Returns a dict of counts over all (sequence, step) positions:
      same      the device's token is the oracle's argmax
      tied      ... or its oracle logit is within 2 bf16 units in the last place of the oracle's largest logit (the
                logits are bf16: two correct bf16 implementations that accumulate in a different order pick different
                tokens among such near-ties)
      decided   positions whose top-1 / top-2 margin exceeds the bf16 error bound of a logit (2e-2 + 3e-2 * the
                row's largest |logit|), and how many of those agree."""
    n_seq, steps = len(prompts), len(produced[0])
    ids = torch.tensor([t for p in prompts for t in p])
    pos = torch.cat([torch.arange(len(p)) for p in prompts])
    logits = oracle.forward(ids, pos, list(range(n_seq)), [len(p) for p in prompts]).float()
    out = dict(n=0, same=0, tied=0, decided=0, decided_same=0, worst_gap_ulps=0.0)
    lens = [len(p) for p in prompts]
    for k in range(steps):
        got = torch.tensor([produced[i][k] for i in range(n_seq)])
        top2 = logits.topk(2, dim=-1)
        best = top2.values[:, 0]
        decided = (best - top2.values[:, 1]) > (2e-2 + 3e-2 * logits.abs().max(-1).values)
        same = got == top2.indices[:, 0]
        ulp = torch.exp2(torch.floor(torch.log2(best.abs().clamp_min(1e-30))) - 7)
        gap_ulps = (best - logits.gather(1, got.view(-1, 1)).squeeze(1)) / ulp
        out["n"] += n_seq
        out["same"] += int(same.sum())
        out["tied"] += int((same | (gap_ulps <= 2.0)).sum())
        out["decided"] += int(decided.sum())
        out["decided_same"] += int(same[decided].sum())
        out["worst_gap_ulps"] = max(out["worst_gap_ulps"], float(gap_ulps.max()))
        if k + 1 < steps:
            logits = oracle.forward(got, torch.tensor(lens), list(range(n_seq)), [1] * n_seq).float()
            lens = [l + 1 for l in lens]
    return out


def test_resident_decoder_step_and_oracle_agree(pkg):
    ensure_group()
    from nanovllm_b200.engine.model_runner import ModelRunner, ResidentDecoder, Seq, sequential_block_tables
    _attention_backend()
    weights = O.init_full_weights(SHAPE, seed=29)
    B, K = 8, 24
    runner = ModelRunner(_config(SHAPE), max_num_seqs=B, max_model_len=1024, max_num_batched_tokens=4096, num_kvcache_blocks=2 * B,
                         oneshot_tokens=256, full_weights=weights)
    try:
        g = torch.Generator().manual_seed(5)
        lens = [37, 250, 5, 256, 257, 100, 64, 300]
        prompts = [torch.randint(0, SHAPE.vocab, (n,), generator=g).tolist() for n in lens]
        tables = sequential_block_tables([512] * B, 256)
        first = runner.step([Seq(list(p), bt) for p, bt in zip(prompts, tables)], True)

        # (a) device-resident loop
        resident = ResidentDecoder(runner, B)
        resident.load([Seq(list(p) + [t], bt) for p, t, bt in zip(prompts, first, tables)])
        via_resident = [[t] for t in first]
        for _ in range(K):
            resident.replay()
            for i, t in enumerate(resident.tokens.tolist()):
                via_resident[i].append(t)
        runner.runtime.check_status()

        # (b) the same steps through step() (host batch state; CUDA-graph replay of the forward)
        seqs = [Seq(list(p) + [t], bt) for p, t, bt in zip(prompts, first, tables)]
        via_step = [[t] for t in first]
        for _ in range(K):
            toks = runner.step(seqs, False)
            for i, (s, t) in enumerate(zip(seqs, toks)):
                s.token_ids.append(t)
                via_step[i].append(t)
        assert via_resident == via_step, "the device-resident loop and step() produced different tokens"

        # (c) the oracle, teacher-forced on those tokens
        oracle = O.QwenOracle(SHAPE, weights, world=1, max_pos=1024)
        r = oracle_agreement(oracle, prompts, via_resident)
        assert r["decided"] > 0 and r["decided_same"] == r["decided"], f"greedy tokens vs the oracle: {r}"
        assert r["tied"] >= 0.99 * r["n"] and r["same"] >= 0.9 * r["n"], f"greedy tokens vs the oracle: {r}"

        # a replay past the loaded blocks is refused on the host ...
        resident.load([Seq(list(range(255)), [0]) for _ in range(B)])
        resident.replay()
        resident.replay()
        with pytest.raises(RuntimeError, match="filled the blocks"):
            resident.replay()
        # ... and on the device a row without room is frozen instead of being sent outside the cache
        from nanovllm_b200 import ops
        gv = runner.graph_vars
        before_pos, before_len = gv["positions"][:B].clone(), gv["context_lens"][:B].clone()
        ops.advance_decode(resident.tokens, gv["input_ids"], gv["positions"], gv["context_lens"], gv["slot_mapping"], gv["block_tables"][:B],
                           runner.block_size, runner.num_kvcache_blocks * runner.block_size)
        torch.cuda.synchronize()
        assert (gv["slot_mapping"][:B] == -1).all() and torch.equal(gv["positions"][:B], before_pos) and torch.equal(gv["context_lens"][:B], before_len)
    finally:
        runner.exit()


def test_chunked_prefill_with_cached_prefix_matches_oracle(pkg):
    ensure_group()
    from nanovllm_b200.engine.model_runner import ModelRunner, Seq, sequential_block_tables
    _attention_backend()
    weights = O.init_full_weights(SHAPE, seed=31)
    runner = ModelRunner(_config(SHAPE), max_num_seqs=8, max_model_len=1024, max_num_batched_tokens=4096, num_kvcache_blocks=16,
                         enforce_eager=True, oneshot_tokens=256, full_weights=weights)
    try:
        g = torch.Generator().manual_seed(9)
        lens = [300, 700, 90]
        # blocks taken from a shuffled free list, as after some traffic
        perm = torch.randperm(16, generator=g).tolist()
        seqs = [Seq(torch.randint(0, SHAPE.vocab, (n,), generator=g).tolist(), bt)
                for n, bt in zip(lens, sequential_block_tables(lens, 256, permutation=perm))]
        oracle = O.QwenOracle(SHAPE, weights, world=1, max_pos=1024)
        ref = oracle.forward(torch.tensor([t for s in seqs for t in s.token_ids]), torch.cat([torch.arange(n) for n in lens]),
                             [0, 1, 2], lens).float()
        # three chunks per sequence: [0, c1), [c1, c2), [c2, len); a chunk boundary inside a block and on a block edge
        cuts = [(100, 256), (256, 513), (1, 89)]
        logits = None
        for chunk in range(3):
            num_new = []
            for s, n, (c1, c2) in zip(seqs, lens, cuts):
                bounds = (0, c1, c2, n)
                s.num_cached_tokens = bounds[chunk]
                num_new.append(bounds[chunk + 1] - bounds[chunk])
            ids, pos = runner.prepare_prefill(seqs, num_new)
            assert ids.numel() == sum(num_new)
            logits = runner.run_model(ids, pos, True).float().cpu()
        runner.runtime.check_status()
        err = (logits - ref).abs().max().item()
        assert err <= 2e-2 + 3e-2 * ref.abs().max().item(), f"chunked prefill: last-token logits differ by {err}"
        top2 = ref.topk(2, dim=-1).values
        decided = (top2[:, 0] - top2[:, 1]) > 2 * err
        assert (logits.argmax(-1) == ref.argmax(-1))[decided].all()
        # the same sequences prefilled in one piece give the same logits up to the kernels' rounding
        for s in seqs:
            s.num_cached_tokens = 0
        ids, pos = runner.prepare_prefill(seqs)
        whole = runner.run_model(ids, pos, True).float().cpu()
        assert (whole - logits).abs().max().item() <= 2e-2 + 3e-2 * ref.abs().max().item()
    finally:
        runner.exit()


@pytest.mark.parametrize("temperature", [None, 0.6])
def test_token_parity_qwen3_0_6b_shape(pkg, temperature):
    """Greedy decoding of a random-init model with Qwen3-0.6B's layer shapes (hidden 1024, 16 q / 8 kv heads of 128,
    MLP 3072, tied embeddings; 4 layers and a 8192-entry vocabulary keep the CPU oracle to a minute): 32 sequences x
    64 decode steps through the device-resident loop, teacher-forced against the oracle.  Reported: identical
    tokens over all positions, the same counting bf16 near-ties of the oracle's own logits as agreement, and the
    decided positions.  (Random-init logits are packed closely: about one position in ten has its two best logits
    within two bf16 units in the last place, and there the argmax depends on the accumulation order.)
    With a temperature the run only checks that sampling runs end to end."""
    ensure_group()
    from nanovllm_b200.engine.model_runner import ModelRunner, ResidentDecoder, Seq, sequential_block_tables
    _attention_backend()
    shape = O.QwenShape(hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, intermediate=3072, n_layers=4, vocab=8192, tie=True)
    weights = O.init_full_weights(shape, seed=41)
    B, K = 32, 64
    if temperature is not None:
        B, K = 16, 8
    runner = ModelRunner(_config(shape), max_num_seqs=B, max_model_len=512, max_num_batched_tokens=4096, num_kvcache_blocks=2 * B,
                         oneshot_tokens=256, full_weights=weights)
    try:
        g = torch.Generator().manual_seed(13)
        prompts = [torch.randint(0, shape.vocab, (int(n),), generator=g).tolist() for n in torch.randint(8, 120, (B,), generator=g)]
        tables = sequential_block_tables([512] * B, 256)
        first = runner.step([Seq(list(p), bt) for p, bt in zip(prompts, tables)], True)
        if temperature is not None:
            seqs = [Seq(list(p) + [t], bt) for p, t, bt in zip(prompts, first, tables)]
            for _ in range(K):
                toks = runner.step(seqs, False, temperatures=[temperature] * B)
                assert len(toks) == B and all(0 <= t < shape.vocab for t in toks)
                for s, t in zip(seqs, toks):
                    s.token_ids.append(t)
            return
        resident = ResidentDecoder(runner, B)
        resident.load([Seq(list(p) + [t], bt) for p, t, bt in zip(prompts, first, tables)])
        produced = [[t] for t in first]
        for _ in range(K):
            resident.replay()
            for i, t in enumerate(resident.tokens.tolist()):
                produced[i].append(t)
        runner.runtime.check_status()
        oracle = O.QwenOracle(shape, weights, world=1, max_pos=512)
        r = oracle_agreement(oracle, prompts, produced)
        print(f"token parity over {r['n']} positions: identical {r['same']}, identical or within 2 bf16 ulps of the oracle's best logit {r['tied']}, "
              f"decided {r['decided_same']}/{r['decided']}, worst gap {r['worst_gap_ulps']:.2f} ulps")
        assert r["decided_same"] == r["decided"], f"a decided position disagrees: {r}"
        assert r["tied"] >= 0.99 * r["n"], f"fewer than 99 % of the positions agree up to bf16 near-ties: {r}"
        assert r["same"] >= 0.95 * r["n"], f"fewer than 95 % of the positions are identical: {r}"
    finally:
        runner.exit()
