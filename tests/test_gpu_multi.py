"""The cross-GPU paths on 2 (and, when present, 4 and 8) B200s: fused
row-parallel GEMM + push + reduce + residual + RMSNorm, embedding broadcast,
LM-head gather, token broadcast, and a small Qwen3 end to end, each rank in
its own process, against the CPU oracle with the same world size."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    entry.load_package()
    from nanovllm_b200 import ops, _abi
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    from oracle import tp_path as O
    from tests.gpu_util import assert_close_bf16, ulp_mismatch_fraction
    dev = torch.device("cuda", rank)
    vocab = 4096 * world
    # every rank computes the CPU oracle of every case: keep the cases small when there are many ranks
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
    big = world <= 2 and os.environ.get("B2_TEST_SMALL_CASES") != "1"
    H = 5120 if big else 1024
    rt = init_runtime(max_tokens=4096, hidden=H, oneshot_tokens=512, vocab=vocab, max_seqs=64)
    try:
        # ---- fused row-parallel block: shapes follow each other without a host sync ----
        if big:
            shapes = [(64, 4096, 4096), (1, 2048, 1024), (8, 8192, H), (64, 12288, 4096), (200, 1024, H), (512, 2048, 1024),
                      (700, 1024, 2048), (64, 4096, 4096), (128, 2048, 1024), (256, 2048, 2048), (96, 6144, 1024)]
        else:
            shapes = [(64, 2048, 1024), (1, 1024, 1024), (8, 2048, H), (200, 1024, H), (512, 1024, 1024), (64, 1024, 512)]
        results = []
        for i, (m, k, n) in enumerate(shapes):
            xs, ws, residual, norm_w = O.rowpar_case(m, k, n, world, seed=100 + i)
            normed, new_res = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
            # (the two-shot form returns a view of a buffer the next two-shot call reuses: keep a copy)
            results.append(((normed.clone(), new_res), xs, ws, residual, norm_w, (m, k, n)))
        torch.cuda.synchronize()
        rt.check_status()
        for (normed, new_res), xs, ws, residual, norm_w, shp in results:
            exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
            assert_close_bf16(normed, exact_n, f"rank {rank} normed {shp}")
            if ops.rowpar_form(shp[0], shp[2]) == _abi.FORM_TWOSHOT:
                # two-shot form: the residual stays with the ranks that own the rows (16-row blocks, round-robin)
                mine = (torch.arange(shp[0]) // 16) % world == rank
                assert_close_bf16(new_res.cpu()[mine], exact_s[mine], f"rank {rank} residual (owned rows) {shp}")
                continue
            assert_close_bf16(new_res, exact_s, f"rank {rank} residual {shp}")
            # the reference rounds the all-reduced sum to bf16 before the residual add; the fused kernel keeps
            # it in fp32, so the two differ by at most that one rounding (2^-8 relative to the summed value)
            ref_n, ref_s = O.fused_row_parallel_norm(xs, ws, residual, norm_w, 1e-6)
            y_max = O.row_parallel_linear(xs, ws).float().abs().max().item()
            assert (new_res.float().cpu() - ref_s.float()).abs().max().item() <= 2 ** -7 * max(y_max, ref_s.float().abs().max().item()), shp
        # every rank holds the same bits (each reduces the same partials in the same order)
        probe = results[0][0][0].float().sum().item()
        gathered = [None] * world
        dist.all_gather_object(gathered, probe)
        assert all(g == gathered[0] for g in gathered), gathered

        # ---- the row-owner form (row t reduced by rank t mod world, finished rows sent to everyone), forced at every size it takes ----
        owner_shapes = [(64, 4096, 4096), (1, 2048, 1024), (8, 8192, H), (5, 1024, H), (63, 1024, 4096), (200, 1024, H), (512, 2048, 1024)] if big \
            else [(64, 2048, 1024), (1, 1024, 1024), (8, 2048, H), (5, 1024, H), (63, 1024, 512), (200, 1024, H), (512, 1024, 1024)]
        for i, (m, k, n) in enumerate(owner_shapes):
            xs, ws, residual, norm_w = O.rowpar_case(m, k, n, world, seed=500 + i)
            args = (xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
            rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, 1 << 20)  # keep the many-token two-shot kernel out of this section
            rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_ONESHOT)
            one_n, one_s = ops.rowpar_fused(*args)
            rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_OWNER)
            for _ in range(3):
                own_n, own_s = ops.rowpar_fused(*args)
            y = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, None, None, 0.0)
            rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
            rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, rt.default_twoshot_min_tokens)
            torch.cuda.synchronize()
            rt.check_status()
            exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
            assert_close_bf16(own_n, exact_n, f"rank {rank} owner form normed {(m, k, n)}")
            assert_close_bf16(own_s, exact_s, f"rank {rank} owner form residual {(m, k, n)}")
            assert_close_bf16(y, sum(x.float() @ w.float().t() for x, w in zip(xs, ws)), f"rank {rank} owner form plain forward {(m, k, n)}")
            if m <= 64:  # same partials (cluster kernel), same summation order: the two forms agree exactly
                assert torch.equal(own_n, one_n) and torch.equal(own_s, one_s), f"rank {rank}: owner and one-shot forms differ {(m, k, n)}"
        # forms alternating launch by launch, many times: the inbox parities stay in step on every rank
        xs, ws, residual, norm_w = O.rowpar_case(64, 1024, 1024, world, seed=12)
        args = (xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
        for i in range(61):
            rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_OWNER if i % 3 else _abi.FORM_ONESHOT)
            normed, new_res = ops.rowpar_fused(*args)
        rt.set_option(_abi.OPT_ROWPAR_FORM, _abi.FORM_AUTO)
        torch.cuda.synchronize()
        rt.check_status()
        assert_close_bf16(normed, O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)[0], "61 launches of alternating forms")

        # ---- two-shot form (many tokens): normed rows everywhere, the residual only on the rows a rank owns ----
        rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, 128)  # this section is about the two-shot kernel: give it these sizes
        for i, (m, k) in enumerate([(1024, 2048), (300, 1024), (4096, 1024), (777, 2048)] if big else [(512, 1024), (300, 1024), (1040, 1024)]):
            n = H
            xs, ws, residual, norm_w = O.rowpar_case(m, k, n, world, seed=300 + i)
            for _ in range(2):
                normed, new_res = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
            torch.cuda.synchronize()
            rt.check_status()
            exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
            assert_close_bf16(normed, exact_n, f"rank {rank} two-shot normed M={m}")
            mine = (torch.arange(m) // 16) % world == rank  # 16-row blocks are dealt round-robin
            assert_close_bf16(new_res.cpu()[mine], exact_s[mine], f"rank {rank} two-shot residual (owned rows)")
            # row-sharded residual feeds the next call: chain a second block on the first one's outputs
            xs2, ws2, _, norm_w2 = O.rowpar_case(m, k, n, world, seed=400 + i)
            normed2, res2 = ops.rowpar_fused(xs2[rank].to(dev), ws2[rank].to(dev), None, new_res, norm_w2.to(dev), 1e-6)
            torch.cuda.synchronize()
            y2 = sum(x.float() @ w.float().t() for x, w in zip(xs2, ws2))
            s2 = y2 + exact_s.bfloat16().float()
            n2 = s2 * torch.rsqrt(s2.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w2.float()
            assert_close_bf16(normed2, n2, f"rank {rank} chained two-shot normed M={m}", abs_tol=4e-2, rel_tol=1e-2)
        y = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, None, None, 0.0)  # plain forward through the two-shot kernel
        assert_close_bf16(y, sum(x.float() @ w.float().t() for x, w in zip(xs, ws)), "two-shot plain forward")
        rt.check_status()
        rt.set_option(_abi.OPT_TWOSHOT_MIN_TOKENS, rt.default_twoshot_min_tokens)

        # ---- plain RowParallelLinear.forward with a bias (added once, by rank 0) ----
        xs, ws, _, _ = O.rowpar_case(48, 1024, 1024, world, seed=7)
        bias = torch.randn(1024, generator=torch.Generator().manual_seed(1)).bfloat16()
        y = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), bias.to(dev), None, None, 0.0)
        assert_close_bf16(y, sum(x.float() @ w.float().t() for x, w in zip(xs, ws)) + bias.float(), "row-parallel forward + bias")

        # ---- many launches back to back: the two inboxes keep alternating cleanly ----
        xs, ws, residual, norm_w = O.rowpar_case(64, 1024, 1024, world, seed=9)
        x_d, w_d, r_d, n_d = xs[rank].to(dev), ws[rank].to(dev), residual.to(dev), norm_w.to(dev)
        for _ in range(101):
            normed, new_res = ops.rowpar_fused(x_d, w_d, None, r_d, n_d, 1e-6)
        torch.cuda.synchronize()
        rt.check_status()
        assert_close_bf16(normed, O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)[0], "101st launch")

        # ---- embedding: the owner rank's rows reach everyone, bit-exact ----
        g = torch.Generator().manual_seed(5)
        table = torch.randn(vocab, 1024, generator=g).bfloat16()
        per = vocab // world
        shard = table[rank * per:(rank + 1) * per].to(dev)
        for m in (1, 64, 700, 2048):
            ids = torch.randint(0, vocab, (m,), generator=g)
            got = ops.embed(ids.to(dev), shard, rank * per, (rank + 1) * per, world)
            torch.cuda.synchronize()
            assert torch.equal(got.cpu(), table[ids]), f"embedding M={m}"
        rt.check_status()

        # ---- LM head: every rank's slice lands in rank 0's [B, vocab] buffer ----
        h = torch.randn(40, 1024, generator=g).bfloat16()
        for idx in (None, torch.tensor([0, 7, 39], dtype=torch.int32)):
            logits = ops.lm_head(h.to(dev), shard, idx.to(dev) if idx is not None else None)
            torch.cuda.synchronize()
            rows = h if idx is None else h[idx.long()]
            if rank == 0:
                assert_close_bf16(logits, rows.float() @ table.float().t(), "gathered logits")
            else:
                assert logits is None
            dist.barrier()  # rank 0 has read the buffer before anyone writes it again
        rt.check_status()

        # ---- LM head fused with the sampler: each rank scans its vocabulary slice, only (score, id) per row travels ----
        from tests.gpu_util import check_sampler_picks
        logits = ops.lm_head(h.to(dev), shard, None)
        torch.cuda.synchronize()
        logits = logits.clone() if rank == 0 else None
        dist.barrier()
        temps = (torch.rand(40, generator=g) + 0.3).to(dev)
        for call, t in enumerate([None, temps, temps, None]):
            buf = torch.full((40,), -7, dtype=torch.int64, device=dev)
            ops.lm_head_sample(h.to(dev), shard, None, t, 99, out=buf)
            ops.broadcast_tokens(buf)            # rank 0's picks to everyone (and the exchange that separates two sampler calls)
            torch.cuda.synchronize()
            if rank == 0:
                check_sampler_picks(buf, logits, t, O.fused_sampler_noise(99, call, 40, vocab) if t is not None else None, f"fused sampler call {call}")
            everyone = [None] * world
            dist.all_gather_object(everyone, buf.tolist())
            assert all(e == everyone[0] for e in everyone), "token broadcast after the fused sampler"
        rt.check_status()

        # ---- token broadcast ----
        for step in range(3):
            buf = (torch.arange(64, device=dev) * (step + 1) + 5) if rank == 0 else torch.zeros(64, dtype=torch.int64, device=dev)
            ops.broadcast_tokens(buf)
            torch.cuda.synchronize()
            assert buf.tolist() == [i * (step + 1) + 5 for i in range(64)]
        rt.check_status()
    finally:
        shutdown_runtime()

    # ---- a small Qwen3 end to end at this world size ----
    from nanovllm_b200.engine.model_runner import ModelConfig, ModelRunner, Seq, sequential_block_tables
    shape = O.QwenShape(hidden=512, n_heads=8, n_kv_heads=8, head_dim=128, intermediate=1024, n_layers=3, vocab=1024 * world)
    weights = O.init_full_weights(shape, seed=23)
    cfg = ModelConfig(hidden_size=shape.hidden, num_attention_heads=shape.n_heads, num_key_value_heads=shape.n_kv_heads, head_dim=shape.head_dim,
                      intermediate_size=shape.intermediate, num_hidden_layers=shape.n_layers, vocab_size=shape.vocab, max_position_embeddings=1024)
    runner = ModelRunner(cfg, max_num_seqs=16, max_model_len=1024, max_num_batched_tokens=2048, num_kvcache_blocks=16,
                         oneshot_tokens=256, full_weights=weights)
    try:
        g = torch.Generator().manual_seed(3)
        lens = [37, 300, 5]
        seqs = [Seq(torch.randint(0, shape.vocab, (n,), generator=g).tolist()) for n in lens]
        for s, bt in zip(seqs, sequential_block_tables([n + 8 for n in lens], 256)):
            s.block_table = bt
        oracle = O.QwenOracle(shape, weights, world=world, max_pos=1024)
        ref = oracle.forward(torch.tensor([t for s in seqs for t in s.token_ids]), torch.cat([torch.arange(n) for n in lens]),
                             [0, 1, 2], lens).float()
        ids, pos = runner.prepare_prefill(seqs)
        logits = runner.run_model(ids, pos, True)
        for step in range(5):
            if rank == 0:
                err = (logits.float().cpu() - ref).abs().max().item()
                assert err <= 2e-2 + 3e-2 * ref.abs().max().item(), f"step {step}: logits differ by {err}"
            else:
                assert logits is None
            nxt = ref.argmax(-1).tolist()
            for s, t in zip(seqs, nxt):
                s.token_ids.append(t)
            ref = oracle.forward(torch.tensor(nxt), torch.tensor([len(s) - 1 for s in seqs]), [0, 1, 2], [1, 1, 1]).float()
            ids, pos = runner.prepare_decode(seqs)
            logits = runner.run_model(ids, pos, False)  # CUDA-graph replay
            dist.barrier()
        toks = runner.step(seqs, False)  # greedy tokens reach every rank
        gathered = [None] * world
        dist.all_gather_object(gathered, toks)
        assert all(t == gathered[0] for t in gathered)
        runner.runtime.check_status()
    finally:
        runner.exit()
        dist.destroy_process_group()


def _timeout_worker(rank: int, world: int, port: int):
    """Failure made on the host: rank 1 never issues its half of a fused call.  Rank 0's kernel waits for the
    partial rows, gives up after the context's limit, reports it through the status word and ends normally."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as entry
    entry.load_package()
    from nanovllm_b200 import ops, _abi
    from nanovllm_b200.runtime import init_runtime, shutdown_runtime
    from oracle import tp_path as O
    dev = torch.device("cuda", rank)
    rt = init_runtime(max_tokens=256, hidden=1024, oneshot_tokens=256, timeout_ms=300)
    try:
        xs, ws, residual, norm_w = O.rowpar_case(16, 1024, 1024, world, seed=1)
        # a healthy call first
        ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
        torch.cuda.synchronize()
        rt.check_status()
        dist.barrier()
        if rank == 0:
            ops.rowpar_fused(xs[0].to(dev), ws[0].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
            torch.cuda.synchronize()  # returns: the wait is bounded
            with pytest.raises(_abi.B2Error, match="partial rows never arrived"):
                rt.check_status()
            # the device is still usable after the expired wait
            assert torch.ones(4, device=dev).sum().item() == 4.0
            # ... but the context is not, until every rank has reset it
            with pytest.raises(_abi.B2Error, match="reset"):
                rt.check_status()
        dist.barrier()  # rank 1 has launched nothing in between
        # rank 0's abandoned partial rows sit in rank 1's inbox and the ranks' launch counters differ by one:
        # the collective reset puts both back, and a healthy call gives the right sums again
        rt.reset()
        from tests.gpu_util import assert_close_bf16
        for _ in range(3):
            normed, new_res = ops.rowpar_fused(xs[rank].to(dev), ws[rank].to(dev), None, residual.to(dev), norm_w.to(dev), 1e-6)
        torch.cuda.synchronize()
        rt.check_status()
        exact_n, exact_s = O.fused_row_parallel_norm_exact(xs, ws, residual, norm_w, 1e-6)
        assert_close_bf16(normed, exact_n, f"rank {rank}: normed after reset")
        assert_close_bf16(new_res, exact_s, f"rank {rank}: residual after reset")
        dist.barrier()
    finally:
        shutdown_runtime()
        dist.destroy_process_group()


def test_expired_wait_is_reported_not_hung():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_timeout_worker, args=(2, 29790), nprocs=2, join=True)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, 29700 + world), nprocs=world, join=True)
