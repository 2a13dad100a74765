"""Generate the golden fixtures in this directory from the reference itself.

Run where the reference source tree is available:

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py --reference <path to nano-vllm>

It imports the reference's own layer classes (nanovllm/layers/*.py) under a
2-rank gloo process group on the CPU, feeds them seeded inputs, and stores
inputs and outputs as small .pt files.  The torch.compile decorators in the
reference are disabled (TORCHDYNAMO_DISABLE=1) so the same source runs eagerly.
The fixtures are what pins the CPU oracle (oracle/tp_path.py) to the reference.
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
WORLD = 2


def cfg1_inputs(block: str, rank: int):
    """BASELINE config 1: Qwen3-0.6B-shaped row-parallel block in fp32, 64 tokens."""
    kr, n = {"o_proj": (1024, 1024), "down_proj": (1536, 1024)}[block]
    g = torch.Generator().manual_seed(1234 + rank + (0 if block == "o_proj" else 100))
    x = torch.randn(64, kr, generator=g)
    w = torch.randn(n, kr, generator=g) * 0.02
    g2 = torch.Generator().manual_seed(99)
    residual = torch.randn(64, n, generator=g2)
    return x, w, residual


def small_bf16_inputs(seed: int, m: int, k: int, n: int):
    g = torch.Generator().manual_seed(seed)
    x_full = torch.randn(m, k, generator=g).bfloat16()
    w_full = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
    residual = torch.randn(m, n, generator=g).bfloat16()
    norm_w = (torch.rand(n, generator=g) + 0.5).bfloat16()
    return x_full, w_full, residual, norm_w


def worker(rank: int, ref_path: str, port: int, out_dir: str):
    sys.path.insert(0, ref_path)
    dist.init_process_group("gloo", f"tcp://127.0.0.1:{port}", world_size=WORLD, rank=rank)
    from nanovllm.layers.linear import (MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear)
    from nanovllm.layers.layernorm import RMSNorm
    from nanovllm.layers.embed_head import VocabParallelEmbedding, ParallelLMHead
    from nanovllm.layers.activation import SiluAndMul
    from nanovllm.layers.rotary_embedding import RotaryEmbedding
    from nanovllm.utils.context import set_context, reset_context

    out: dict[str, torch.Tensor] = {}

    def gather_to_rank0(t: torch.Tensor) -> list[torch.Tensor]:
        lst = [torch.empty_like(t) for _ in range(WORLD)]
        dist.all_gather(lst, t.contiguous())
        return lst

    with torch.inference_mode():
        # ---- config 1: fp32 row-parallel + add-RMSNorm, TP=2 ----------------
        torch.set_default_dtype(torch.float32)
        for block in ("o_proj", "down_proj"):
            x, w, residual = cfg1_inputs(block, rank)
            layer = RowParallelLinear(w.shape[1] * WORLD, w.shape[0])
            layer.weight.data.copy_(w)
            norm = RMSNorm(w.shape[0], eps=1e-6)
            y = layer(x.clone())
            out[f"cfg1/{block}/y"] = y.clone()
            # fp32 quirk of the reference: the returned residual aliases the
            # normed output, so only the normed output is kept
            normed, _ = norm(y.clone(), residual.clone())
            out[f"cfg1/{block}/normed"] = normed.clone()

        # ---- bf16: row-parallel through the weight loader + add-RMSNorm -----
        torch.set_default_dtype(torch.bfloat16)
        for name, (seed, m, k, n) in {"rp_a": (7, 16, 256, 128), "rp_b": (8, 5, 512, 384)}.items():
            x_full, w_full, residual, norm_w = small_bf16_inputs(seed, m, k, n)
            layer = RowParallelLinear(k, n)
            layer.weight.weight_loader(layer.weight, w_full)
            norm = RMSNorm(n, eps=1e-6)
            norm.weight.data.copy_(norm_w)
            kr = k // WORLD
            x = x_full[:, rank * kr:(rank + 1) * kr].contiguous()
            y = layer(x)
            normed, new_res = norm(y, residual)
            plain = norm(y)
            for key, val in dict(x_full=x_full, w_full=w_full, residual=residual, norm_w=norm_w, y=y, normed=normed, new_res=new_res, plain_norm=plain).items():
                out[f"{name}/{key}"] = val.clone()
            shards = gather_to_rank0(layer.weight.data)
            for r, s in enumerate(shards):
                out[f"{name}/w_shard{r}"] = s.clone()

        # ---- bf16: qkv and merged column-parallel ---------------------------
        g = torch.Generator().manual_seed(21)
        hidden, hd, nh, nkv, inter, m = 128, 32, 8, 4, 192, 9
        xq = torch.randn(m, hidden, generator=g).bfloat16()
        wq = (torch.randn(nh * hd, hidden, generator=g) * 0.05).bfloat16()
        wk = (torch.randn(nkv * hd, hidden, generator=g) * 0.05).bfloat16()
        wv = (torch.randn(nkv * hd, hidden, generator=g) * 0.05).bfloat16()
        wg = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        wu = (torch.randn(inter, hidden, generator=g) * 0.05).bfloat16()
        qkv = QKVParallelLinear(hidden, hd, nh, nkv)
        for sid, t in (("q", wq), ("k", wk), ("v", wv)):
            qkv.weight.weight_loader(qkv.weight, t, sid)
        gu = MergedColumnParallelLinear(hidden, [inter, inter])
        for sid, t in ((0, wg), (1, wu)):
            gu.weight.weight_loader(gu.weight, t, sid)
        yq = qkv(xq)
        yg = gu(xq)
        act = SiluAndMul()(yg)
        out.update({"col/x": xq, "col/wq": wq, "col/wk": wk, "col/wv": wv, "col/wg": wg, "col/wu": wu})
        for r, (a, b, c, d, e) in enumerate(zip(gather_to_rank0(qkv.weight.data), gather_to_rank0(yq), gather_to_rank0(gu.weight.data), gather_to_rank0(yg), gather_to_rank0(act))):
            out[f"col/qkv_w{r}"], out[f"col/qkv_y{r}"] = a.clone(), b.clone()
            out[f"col/gu_w{r}"], out[f"col/gu_y{r}"], out[f"col/act{r}"] = c.clone(), d.clone(), e.clone()

        # ---- bf16: vocab-parallel embedding and LM head ---------------------
        g = torch.Generator().manual_seed(33)
        vocab, hidden = 64, 48
        emb_w = torch.randn(vocab, hidden, generator=g).bfloat16()
        ids = torch.randint(0, vocab, (23,), generator=g)
        emb = VocabParallelEmbedding(vocab, hidden)
        emb.weight.weight_loader(emb.weight, emb_w)
        e = emb(ids)
        head = ParallelLMHead(vocab, hidden)
        head.weight.weight_loader(head.weight, emb_w)
        hs = torch.randn(23, hidden, generator=g).bfloat16()
        set_context(False)
        logits_decode = head(hs)
        cu = torch.tensor([0, 5, 6, 17, 23], dtype=torch.int32)
        set_context(True, cu_seqlens_q=cu)
        logits_prefill = head(hs)
        reset_context()
        out.update({"vocab/w": emb_w, "vocab/ids": ids, "vocab/emb": e.clone(), "vocab/h": hs, "vocab/cu_seqlens_q": cu})
        if rank == 0:
            out["vocab/logits_decode"] = logits_decode.clone()
            out["vocab/logits_prefill"] = logits_prefill.clone()
        else:
            assert logits_decode is None and logits_prefill is None

        # ---- bf16: RoPE and head-dim RMSNorm (rank-independent) --------------
        g = torch.Generator().manual_seed(44)
        rope = RotaryEmbedding(64, 64, 512, 1e6)
        pos = torch.randint(0, 512, (11,), generator=g)
        q = torch.randn(11, 4, 64, generator=g).bfloat16()
        k = torch.randn(11, 2, 64, generator=g).bfloat16()
        hn = RMSNorm(64, eps=1e-6)
        hn.weight.data.copy_((torch.rand(64, generator=g) + 0.5).bfloat16())
        qn = hn(q)
        q2, k2 = rope(pos, q, k)
        out.update({"rope/pos": pos, "rope/q": q, "rope/k": k, "rope/q_out": q2.clone(), "rope/k_out": k2.clone(),
                    "rope/cache": rope.cos_sin_cache.squeeze(1).clone(), "rope/norm_w": hn.weight.data.clone(), "rope/q_normed": qn.clone()})

        # ---- the sampler (the reference runs it on rank 0; the CPU generator is seeded, and the noise it is
        #      about to draw is recorded by drawing the same tensor from the same seed first) ----------------
        from nanovllm.layers.sampler import Sampler
        g = torch.Generator().manual_seed(45)
        logits = (torch.randn(12, 2048, generator=g) * 3).bfloat16()
        temps = torch.tensor([0.3, 0.6, 0.6, 0.8, 1.0, 1.0, 1.2, 1.5, 0.05, 2.0, 0.7, 0.9])
        torch.manual_seed(777)
        noise = torch.empty(12, 2048).exponential_(1)
        torch.manual_seed(777)
        tokens = Sampler()(logits.clone(), temps)
        out.update({"sampler/logits": logits, "sampler/temperatures": temps, "sampler/noise": noise, "sampler/tokens": tokens.clone()})

    dist.barrier()
    if rank == 0:
        groups: dict[str, dict[str, torch.Tensor]] = {}
        for key, val in out.items():
            grp, _, rest = key.partition("/")
            groups.setdefault(grp, {})[rest] = val.detach().clone()
        for grp, d in groups.items():
            torch.save(d, os.path.join(out_dir, f"{grp}.pt"))
            print(grp, sum(v.numel() * v.element_size() for v in d.values()), "bytes")
    dist.destroy_process_group()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--port", type=int, default=29611)
    a = ap.parse_args()
    mp.spawn(worker, args=(a.reference, a.port, HERE), nprocs=WORLD, join=True)
