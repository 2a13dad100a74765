"""Host-side logic that needs no GPU: the stream-K work partition (a Python
model of the arithmetic in csrc/b2_gemm.cu), and the layer classes' weight
sharding at world size 1 and, under gloo, 2."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tp_path as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- stream-K partition ------------------------------------------------------
class Partition:
    def __init__(self, units, ctas):
        self.base, self.rem = divmod(units, ctas)

    def u0(self, c):
        return c * self.base + min(c, self.rem)

    def cta_of(self, u):
        big = self.rem * (self.base + 1)
        return u // (self.base + 1) if u < big else self.rem + (u - big) // self.base


def gemm_ctas(units, sms=148):
    return max(1, min(sms, units, max(1, units // 8)))


def segments(p, c, kb):
    u, end, out = p.u0(c), p.u0(c + 1), []
    while u < end:
        tile, k0 = divmod(u, kb)
        ln = min(kb - k0, end - u)
        out.append((tile, k0, k0 + ln))
        u += ln
    return out


@pytest.mark.parametrize("tiles,kb", [(1, 1), (32, 64), (32, 192), (48, 64), (192, 64), (1187, 64), (1280, 16), (3, 5), (7, 400), (200, 3)])
def test_streamk_partition_covers_every_unit_once(tiles, kb):
    units = tiles * kb
    g = gemm_ctas(units)
    p = Partition(units, g)
    assert p.u0(g) == units and p.base >= 1
    seen = [0] * units
    slots_used = {}
    for c in range(g):
        segs = segments(p, c, kb)
        for u in range(p.u0(c), p.u0(c + 1)):
            assert p.cta_of(u) == c
        for i, (tile, k0, k1) in enumerate(segs):
            for k in range(k0, k1):
                seen[tile * kb + k] += 1
        partial = [s for s in segs if not (s[1] == 0 and s[2] == kb)]
        assert len(partial) <= 2
    assert all(v == 1 for v in seen)
    # contributors of a tile = CTAs from cta_of(first unit) to cta_of(last unit)
    for tile in range(min(tiles, 64)):
        first, last = p.cta_of(tile * kb), p.cta_of(tile * kb + kb - 1)
        who = sorted({c for c in range(g) for (t, _, _) in segments(p, c, kb) if t == tile})
        assert who == list(range(first, last + 1))
    # a split tile accumulates in the slot of its first contributor: no two split tiles share one
    owners = [p.cta_of(t * kb) for t in range(tiles) if p.cta_of(t * kb) != p.cta_of(t * kb + kb - 1)]
    assert len(owners) == len(set(owners))


# ---- weight loaders ------------------------------------------------------------
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


# ---- two-shot ownership of token rows (owner_of / owned_rows in csrc/b2_gemm.cu) ----
def owner_of(token, world):
    b = token >> 4
    return b % world, ((b // world) << 4) + (token & 15)


def owned_rows(m, world, rank):
    blocks = (m + 15) >> 4
    mine = (blocks - rank + world - 1) // world
    if mine <= 0:
        return 0
    last_block = rank + (mine - 1) * world
    last_rows = m - (last_block << 4) if last_block == blocks - 1 else 16
    return (mine - 1) * 16 + last_rows


@pytest.mark.parametrize("m", [1, 15, 16, 17, 128, 200, 300, 777, 1024, 4096, 16384])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_shot_row_ownership(m, world):
    per_rank = {r: [] for r in range(world)}
    for t in range(m):
        o, l = owner_of(t, world)
        per_rank[o].append(l)
    for r in range(world):
        n = owned_rows(m, world, r)
        # the owner's local rows are exactly 0 .. n-1, each once: the reduce phase walks them as a dense range
        assert sorted(per_rank[r]) == list(range(n)), (m, world, r)
        # and the reduce phase's inverse map (local row -> token) lands on this rank's tokens
        for row in range(n):
            token = (((row >> 4) * world + r) << 4) + (row & 15)
            assert token < m and owner_of(token, world) == (r, row)
    assert sum(owned_rows(m, world, r) for r in range(world)) == m
    # the inbox is sized for the rank that owns most
    max_rows = ((16384 + 15) // 16 + world - 1) // world * 16
    assert max(owned_rows(min(m, 16384), world, r) for r in range(world)) <= max_rows


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
