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
