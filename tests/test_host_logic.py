"""Host-side logic that needs no GPU: the GEMM launch planner and the two-shot row
ownership (the library's own arithmetic, read through its b2_plan_* entry
points), and the layer classes' weight sharding at world size 1 and, under gloo, 2."""
import ctypes as C
import os

import pytest
from hypothesis import given, settings, strategies as st
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tp_path as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- the GEMM launch planner (the library's own arithmetic, read through b2_plan_gemm) ----
EPI_STORE, EPI_PUSH, EPI_PUSH2, EPI_SAMPLE, EPI_PUSH3 = 0, 1, 2, 3, 4
SMS = 148
# clusters of S CTAs resident at once, per tile width: [S] for 32-token tiles, [9 + S] for 64-token tiles.  On a GPU
# the library asks the occupancy calculator; these stand for a 148-SM part whose clusters of 3, 5, 6 and 7 pack badly
RESIDENT = [0, 148, 74, 44, 37, 26, 22, 18, 18] + [0, 148, 74, 44, 37, 26, 22, 18, 18]


def plan_gemm(abi, epi, m, n, k, sms=SMS, resident=RESIDENT):
    plan = abi.GemmPlan()
    res = (C.c_int * 18)(*resident) if resident is not None else None
    rc = abi.lib.b2_plan_gemm(epi, m, n, k, sms, res, C.byref(plan))
    return rc, plan


def plan_gemm_opts(abi, epi, m, n, k, options, sms=SMS):
    plan = abi.GemmPlan()
    rc = abi.lib.b2_plan_gemm_opts(epi, m, n, k, sms, (C.c_int * 18)(*RESIDENT), options, C.byref(plan))
    return rc, plan


def cta_units(abi, plan, cta):
    cap = 4096
    buf = (C.c_int * (3 * cap))()
    n = abi.lib.b2_plan_cta_units(C.byref(plan), cta, buf, cap)
    assert n >= 0, f"producer and consumer walks disagree (code {-n})"
    if n > cap:
        cap = n
        buf = (C.c_int * (3 * cap))()
        assert abi.lib.b2_plan_cta_units(C.byref(plan), cta, buf, cap) == n
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


def check_plan(abi, plan, m, n, k):
    """Every K block of every output tile is computed exactly once, by the CTAs the combine step expects."""
    tiles = plan.tiles_p * plan.tiles_q
    rows_p, rows_q = (n, m) if plan.swap else (m, n)
    assert plan.tiles_p * 128 >= rows_p > (plan.tiles_p - 1) * 128
    assert plan.tiles_q * plan.bn >= rows_q > (plan.tiles_q - 1) * plan.bn
    assert plan.kblocks * 64 >= k > (plan.kblocks - 1) * 64
    assert 1 <= plan.gemm_ctas <= plan.grid and (plan.grid <= SMS or (plan.cluster_split == 1 and plan.grid <= 4 * SMS))
    seen = {}
    holders = {}
    for cta in range(plan.grid):
        units = cta_units(abi, plan, cta)
        if cta >= plan.gemm_ctas:
            assert units == []
        segs = 0
        for i, (tile, kb, starts) in enumerate(units):
            assert 0 <= tile < tiles and 0 <= kb < plan.kblocks
            assert (tile, kb) not in seen, f"unit {(tile, kb)} computed by CTAs {seen[(tile, kb)]} and {cta}"
            seen[(tile, kb)] = cta
            holders.setdefault(tile, set()).add(cta)
            if i > 0 and not starts:      # inside a segment: same tile, next K block (one accumulator, one commit)
                assert (tile, kb) == (units[i - 1][0], units[i - 1][1] + 1)
            else:
                assert starts == 1
            segs += starts
        if plan.cluster_split == 0 and not plan.round_robin:
            partial = sum(1 for t in {u[0] for u in units} if sum(1 for u in units if u[0] == t) < plan.kblocks)
            assert partial <= 2           # a contiguous range cuts at most the tiles at its two ends
    assert len(seen) == tiles * plan.kblocks
    first, last = C.c_int(), C.c_int()
    split_slots = []
    for tile in range(tiles):
        assert abi.lib.b2_plan_tile_contributors(C.byref(plan), tile, C.byref(first), C.byref(last)) == 0
        assert sorted(holders[tile]) == list(range(first.value, last.value + 1)) or plan.round_robin
        if plan.round_robin:
            assert holders[tile] == {first.value} and first.value == last.value
        if first.value != last.value and plan.cluster_split == 0:
            split_slots.append(first.value)
    # a split tile accumulates in the workspace slot of its first contributor: no two split tiles may share one
    assert len(split_slots) == len(set(split_slots))


PLAN_SHAPES = [
    # (epilogue, M, N, K)                       what it is
    (EPI_STORE, 64, 6144, 4096),                # qkv, Qwen3-8B decode, TP=1: cluster kernel
    (EPI_STORE, 64, 24576, 4096),               # gate_up: 192 tiles > 148 SMs -> stream-K
    (EPI_STORE, 64, 151936, 4096),              # LM head: 1187 tiles
    (EPI_STORE, 1, 768, 4096), (EPI_STORE, 8, 4096, 512), (EPI_STORE, 33, 3072, 1024),
    (EPI_STORE, 200, 1024, 4096), (EPI_STORE, 256, 12288, 4096),
    (EPI_STORE, 257, 4096, 4096), (EPI_STORE, 4096, 4096, 4096), (EPI_STORE, 16384, 6144, 4096), (EPI_STORE, 1000, 40, 72),
    (EPI_PUSH, 64, 4096, 4096), (EPI_PUSH, 64, 5120, 1024), (EPI_PUSH, 64, 5120, 3200), (EPI_PUSH, 256, 5120, 1024), (EPI_PUSH, 1, 1024, 384),
    (EPI_PUSH2, 128, 5120, 1024), (EPI_PUSH2, 1024, 5120, 3200), (EPI_PUSH2, 8192, 5120, 1024), (EPI_PUSH2, 16384, 4096, 2048),
    (EPI_PUSH2, 300, 1024, 1536),
    (EPI_PUSH3, 64, 4096, 512), (EPI_PUSH3, 64, 4096, 1536), (EPI_PUSH3, 1, 5120, 1024), (EPI_PUSH3, 8, 5120, 3200), (EPI_PUSH3, 64, 5120, 3200),
    (EPI_PUSH3, 65, 5120, 1024), (EPI_PUSH3, 256, 5120, 1024), (EPI_PUSH3, 1024, 5120, 3200), (EPI_PUSH3, 200, 1024, 384),
    (EPI_SAMPLE, 64, 151936, 4096), (EPI_SAMPLE, 64, 18992, 4096), (EPI_SAMPLE, 256, 4096, 1024), (EPI_SAMPLE, 3, 512, 128),
]


@pytest.mark.parametrize("epi,m,n,k", PLAN_SHAPES)
def test_planner_covers_every_unit_once(pkg, epi, m, n, k):
    from nanovllm_b200 import _abi
    rc, plan = plan_gemm(_abi, epi, m, n, k)
    assert rc == 0
    assert plan.swap == (1 if (epi != EPI_PUSH2 and m <= (64 if epi == EPI_PUSH3 else 256)) else 0)
    if epi == EPI_PUSH2:
        assert plan.grid == SMS and plan.cluster_split == 0
    if epi == EPI_PUSH3:   # decode sizes run in the cluster kernel (its CTAs also reduce and collect); above, stream-K on all SMs
        assert (plan.cluster_split > 0 and plan.grid == plan.gemm_ctas) if m <= 64 else (plan.cluster_split == 0 and plan.grid == SMS)
    if epi == EPI_SAMPLE:
        assert plan.cluster_split == 0 and plan.tiles_q == 1      # the fused sampler runs in the stream-K kernel, one token tile
    check_plan(_abi, plan, m, n, k)


def test_planner_choices_for_the_decode_shapes(pkg):
    """The choices the measured numbers rest on: decode GEMMs of at most one wave of tiles go to the cluster kernel
    with the largest K split that stays resident; 192 tiles go to stream-K on all SMs; prefill walks whole tiles."""
    from nanovllm_b200 import _abi
    rc, p = plan_gemm(_abi, EPI_STORE, 64, 6144, 4096)           # 48 tiles: 3 CTAs per tile would fit 148 SMs but
    assert (p.bn, p.tiles_p, p.cluster_split) == (64, 48, 2)      # only 44 such clusters are resident -> split 2
    assert p.grid == p.gemm_ctas == 96
    rc, p = plan_gemm(_abi, EPI_STORE, 64, 4096, 4096)           # 32 tiles: split 4 (37 resident)
    assert (p.tiles_p, p.cluster_split, p.grid) == (32, 4, 128)
    rc, p = plan_gemm(_abi, EPI_STORE, 64, 24576, 4096)
    assert (p.cluster_split, p.gemm_ctas, p.round_robin, p.bn) == (0, 148, 0, 64)
    rc, p = plan_gemm(_abi, EPI_STORE, 64, 6144, 4096, resident=None)   # cluster kernel switched off
    assert (p.cluster_split, p.gemm_ctas) == (0, 148)
    rc, p = plan_gemm(_abi, EPI_STORE, 16384, 4096, 4096)
    assert (p.swap, p.bn, p.round_robin, p.gemm_ctas) == (0, 256, 1, 148)
    rc, p = plan_gemm(_abi, EPI_STORE, 16, 64, 64)                # one unit: one CTA
    assert (p.gemm_ctas, p.grid) == (1, 1)
    rc, p = plan_gemm(_abi, EPI_PUSH, 300, 64, 64)                # one-shot, stream-K kernel: one CTA has GEMM work, but
    assert (p.cluster_split, p.gemm_ctas, p.grid) == (0, 1, 148)  # the launch keeps CTAs for the reduce phase (one per row, at most all SMs)
    rc, p = plan_gemm(_abi, EPI_STORE, 256, 4096, 1024)           # 65..256 tokens: 64-token tiles on the cluster kernel when every
    assert (p.bn, p.tiles_p, p.tiles_q, p.cluster_split, p.grid) == (64, 32, 4, 1, 128)   # (feature tile, token tile) pair fits one wave
    rc, p = plan_gemm(_abi, EPI_STORE, 128, 1024, 2048)
    assert (p.bn, p.tiles_p, p.tiles_q, p.cluster_split, p.grid) == (64, 8, 2, 8, 128)
    rc, p = plan_gemm(_abi, EPI_STORE, 256, 6144, 4096)           # 48 x 4 pairs do not fit one wave and K is long: stream-K as before
    assert (p.bn, p.cluster_split) == (256, 0)
    rc, p = plan_gemm(_abi, EPI_STORE, 256, 6144, 1024)           # short K: unsplit tiles in two waves (a plain GEMM's CTAs wait for nobody)
    assert (p.bn, p.tiles_q, p.cluster_split, p.grid) == (64, 4, 1, 192)
    rc, p = plan_gemm(_abi, EPI_PUSH, 256, 6144, 1024)            # a fused call's CTAs wait for each other: one wave or stream-K
    assert p.cluster_split == 0
    rc, p = plan_gemm(_abi, EPI_PUSH, 64, 5120, 1024)             # one-shot at decode size: the cluster kernel reduces too
    assert (p.tiles_p, p.cluster_split, p.grid) == (40, 3, 120)
    rc, p = plan_gemm(_abi, EPI_PUSH3, 64, 4096, 512)             # row-owner form, o_proj of Qwen3-8B at 8 ranks: 32 tiles x split 4
    assert (p.tiles_p, p.cluster_split, p.grid) == (32, 4, 128)
    for bad in [(0, 0, 64, 64), (0, 64, 0, 64), (0, 64, 64, 0), (5, 64, 64, 64), (-1, 64, 64, 64)]:
        assert plan_gemm(_abi, *bad)[0] == 1                      # B2_ERR_ARG
    assert _abi.lib.b2_plan_gemm(0, 64, 64, 64, SMS, None, None) == 1


@pytest.mark.parametrize("epi,m,n,k", [(EPI_PUSH2, 256, 5120, 1024), (EPI_PUSH2, 512, 5120, 3200), (EPI_STORE, 300, 4096, 4096), (EPI_PUSH3, 256, 5120, 12800),
                                       (EPI_PUSH2, 1024, 5120, 1024), (EPI_STORE, 8192, 5120, 1024)])
def test_whole_tile_option(pkg, epi, m, n, k):
    """Planner option 1 (B2_OPT_WHOLE_TILES): a many-token problem that fits one wave of tiles at some tile width gets one
    whole tile per CTA - nothing is split, so no fp32 combine - and everything else is planned as before."""
    from nanovllm_b200 import _abi
    rc, base = plan_gemm(_abi, epi, m, n, k)
    rc2, opt = plan_gemm_opts(_abi, epi, m, n, k, 1)
    assert rc == 0 and rc2 == 0
    check_plan(_abi, opt, m, n, k)
    row_tiles = (m + 127) // 128
    fits = [bn for bn in (64, 128, 256) if bn <= base.bn and row_tiles * ((n + bn - 1) // bn) <= SMS]
    if base.swap or not fits or (k + 63) // 64 > 96:   # (a long K range is never given to one CTA alone)
        assert [getattr(opt, f) for f, _ in opt._fields_] == [getattr(base, f) for f, _ in base._fields_]
    else:
        assert opt.bn == fits[0] and opt.round_robin == 1 and opt.gemm_ctas == opt.tiles_p * opt.tiles_q
        for cta in range(opt.gemm_ctas):
            units = cta_units(_abi, opt, cta)
            assert [u[:2] for u in units] == [(cta, kb) for kb in range(opt.kblocks)]


@settings(max_examples=120, deadline=None)
@given(epi=st.sampled_from([EPI_STORE, EPI_PUSH, EPI_PUSH2, EPI_SAMPLE, EPI_PUSH3]), m=st.integers(1, 3000), n8=st.integers(1, 1200), k8=st.integers(1, 700),
       sms=st.sampled_from([148, 132, 7, 1]))
def test_planner_property(epi, m, n8, k8, sms):
    import __graft_entry__
    __graft_entry__.load_package()
    from nanovllm_b200 import _abi
    rc, plan = plan_gemm(_abi, epi, m, n8 * 8, k8 * 8, sms=sms, resident=[0, sms, sms // 2, sms // 3, sms // 4, sms // 5, sms // 6, sms // 7, sms // 8] * 2)
    assert rc == 0
    tiles = plan.tiles_p * plan.tiles_q
    seen = set()
    for cta in range(plan.grid):
        for (tile, kb, _) in cta_units(_abi, plan, cta):
            assert (tile, kb) not in seen
            seen.add((tile, kb))
    assert len(seen) == tiles * plan.kblocks
    assert plan.gemm_ctas <= plan.grid <= max(sms, plan.gemm_ctas)
    if epi != EPI_STORE:
        assert plan.grid <= sms or plan.cluster_split == 0   # launches whose CTAs wait for each other fit one wave


def _golden(name):
    return torch.load(os.path.join(ROOT, "tests", "golden", name + ".pt"))


def _loader_worker(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        entry.load_package()
        from nanovllm_b200.layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear
        from nanovllm_b200.layers.embed_head import VocabParallelEmbedding
        torch.set_default_dtype(torch.bfloat16)
        col, rp, voc = _golden("col"), _golden("rp_b"), _golden("vocab")
        qkv = QKVParallelLinear(128, 32, 8, 4)
        for sid in "qkv":
            qkv.weight.weight_loader(qkv.weight, col["w" + sid], sid)
        gu = MergedColumnParallelLinear(128, [192, 192])
        gu.weight.weight_loader(gu.weight, col["wg"], 0)
        gu.weight.weight_loader(gu.weight, col["wu"], 1)
        row = RowParallelLinear(512, 384)
        row.weight.weight_loader(row.weight, rp["w_full"])
        emb = VocabParallelEmbedding(64, 48)
        emb.weight.weight_loader(emb.weight, voc["w"])
        ok = True
        if world == 2:  # the reference's own shards, from the fixtures
            ok &= torch.equal(qkv.weight.data, col[f"qkv_w{rank}"])
            ok &= torch.equal(gu.weight.data, col[f"gu_w{rank}"])
            ok &= torch.equal(row.weight.data, rp[f"w_shard{rank}"])
        ok &= torch.equal(qkv.weight.data, O.shard_qkv(col["wq"], col["wk"], col["wv"], rank, world))
        ok &= torch.equal(gu.weight.data, O.shard_merged([col["wg"], col["wu"]], rank, world))
        # the paired layout (rows interleaved by the loader, no second copy) holds the same shard
        gu2 = MergedColumnParallelLinear(128, [192, 192]).pair_rows()
        gu2.weight.weight_loader(gu2.weight, col["wg"], 0)
        gu2.weight.weight_loader(gu2.weight, col["wu"], 1)
        ok &= torch.equal(gu2.reference_weight(), gu.weight.data)
        ok &= torch.equal(gu2.paired_weight(), gu.paired_weight()) and gu2.paired_weight().data_ptr() == gu2.weight.data_ptr()
        ok &= torch.equal(row.weight.data, O.shard_row(rp["w_full"], rank, world))
        ok &= torch.equal(emb.weight.data, O.shard_column(voc["w"], rank, world))
        ok &= (qkv.tp_rank, qkv.tp_size, qkv.num_heads, qkv.num_kv_heads) == (rank, world, 8 // world, 4 // world)
        ok &= (emb.vocab_start_idx, emb.vocab_end_idx) == (rank * 64 // world, (rank + 1) * 64 // world)
        # every rank agrees on the result through a real collective
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        q.put((rank, bool(flag.item())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2])
def test_weight_loaders_shard_like_the_reference(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + world
    procs = [ctx.Process(target=_loader_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok in results), results


def test_layers_fail_loudly_without_cuda(pkg):
    """There is no CPU fallback: the runtime refuses to start without a GPU."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from nanovllm_b200.runtime import TPRuntime
    with pytest.raises(RuntimeError, match="CUDA"):
        TPRuntime(0, 1, 0, 16, 64)


# ---- two-shot ownership of token rows (the library's own owner_of / owned_rows, through b2_row_owner / b2_owned_rows) ----
@pytest.mark.parametrize("m", [1, 15, 16, 17, 128, 200, 300, 777, 1024, 4096, 16384])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_two_shot_row_ownership(pkg, m, world):
    from nanovllm_b200 import _abi
    lib = _abi.lib

    def owner_of(t):
        local = C.c_int()
        return lib.b2_row_owner(t, world, C.byref(local)), local.value

    per_rank = {r: [] for r in range(world)}
    for t in range(m):
        o, l = owner_of(t)
        per_rank[o].append(l)
    for r in range(world):
        n = lib.b2_owned_rows(m, world, r)
        # the owner's local rows are exactly 0 .. n-1, each once: the reduce phase walks them as a dense range
        assert sorted(per_rank[r]) == list(range(n)), (m, world, r)
        # and the reduce phase's inverse map (local row -> token) lands on this rank's tokens
        for row in range(n):
            token = (((row >> 4) * world + r) << 4) + (row & 15)
            assert token < m and owner_of(token) == (r, row)
    assert sum(lib.b2_owned_rows(m, world, r) for r in range(world)) == m
    # the inbox is sized for the rank that owns most
    max_rows = ((16384 + 15) // 16 + world - 1) // world * 16
    assert max(lib.b2_owned_rows(min(m, 16384), world, r) for r in range(world)) <= max_rows
    assert lib.b2_owned_rows(m, world, world) < 0 and lib.b2_row_owner(-1, world, C.byref(C.c_int())) < 0


# ---- row-owner form for few tokens: row t belongs to rank t mod world ----
@pytest.mark.parametrize("m", [1, 3, 7, 8, 9, 63, 64, 65, 200, 1024])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_owner_form_row_ownership(pkg, m, world):
    from nanovllm_b200 import _abi
    lib = _abi.lib
    per_rank = {r: [] for r in range(world)}
    for t in range(m):
        local = C.c_int()
        o = lib.b2_owner_form_row(t, world, C.byref(local))
        assert (o, local.value) == (t % world, t // world)
        per_rank[o].append(local.value)
    for r in range(world):
        n = lib.b2_owner_form_rows(m, world, r)
        assert per_rank[r] == list(range(n))          # dense local rows: the reduce phase walks 0 .. n-1, token = row * world + rank
        assert all(row * world + r < m for row in range(n))
        assert n <= (1024 + world - 1) // world         # the inbox holds ceil(oneshot_tokens / world) rows per source
    assert sum(lib.b2_owner_form_rows(m, world, r) for r in range(world)) == m
    assert lib.b2_owner_form_rows(m, world, world) < 0 and lib.b2_owner_form_row(-1, world, C.byref(C.c_int())) < 0


# ---- cluster kernel: 4-column groups of the accumulator dealt round-robin to the S CTAs of a cluster ----
@pytest.mark.parametrize("bn", [32, 64])
@pytest.mark.parametrize("s_", [1, 2, 3, 4, 5, 6, 7, 8])
def test_cluster_group_distribution(bn, s_):
    groups = bn // 4
    gl = (groups + s_ - 1) // s_
    owned = {}
    for crank in range(s_):
        for l in range(gl):
            g = l * s_ + crank
            if g < groups:
                assert g not in owned
                owned[g] = (crank, l)
    assert sorted(owned) == list(range(groups))            # every group has exactly one owner
    assert s_ * gl <= groups + 8                            # the receive buffer [source][local group] is large enough
    for g, (crank, l) in owned.items():                     # sender-side rule: owner = g % S, local index = g / S
        assert (g % s_, g // s_) == (crank, l)
    # tokens of the rows a CTA stores: local token lt = l*4 + j  <->  token (l*S + crank)*4 + j
    tokens = sorted((((lt >> 2) * s_ + crank) << 2) + (lt & 3) for crank in range(s_) for lt in range(gl * 4)
                    if (lt >> 2) * s_ + crank < groups)
    assert tokens == list(range(bn))
