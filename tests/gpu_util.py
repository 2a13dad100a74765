"""Helpers shared by the GPU tests."""
import os

import numpy as np
import torch
import torch.distributed as dist

TOL_ABS, TOL_REL = 2e-2, 1e-2  # the bf16 tolerance of the path: |err| <= 2e-2 + 1e-2 * max|ref| against an fp32 reference


def ensure_group():
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("gloo", rank=0, world_size=1)


def assert_close_bf16(got: torch.Tensor, ref_fp32: torch.Tensor, what: str = "", abs_tol=TOL_ABS, rel_tol=TOL_REL):
    got = got.float().cpu()
    ref = ref_fp32.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    if ref.numel() == 0:
        return
    err = (got - ref).abs()
    bound = abs_tol + rel_tol * ref.abs().max().item()
    worst = err.max().item() if err.numel() else 0.0
    if not worst <= bound:
        idx = np.unravel_index(int(err.argmax()), err.shape)
        bad = (err > bound).float().mean().item()
        raise AssertionError(f"{what}: max abs err {worst:.4e} > {bound:.4e} at {idx} (got {got[idx].item():.5f}, ref {ref[idx].item():.5f}); "
                             f"{bad * 100:.2f}% of elements out of tolerance")


def ulp_mismatch_fraction(got: torch.Tensor, ref: torch.Tensor, ulps: int = 1) -> float:
    """Fraction of bf16 elements that differ by more than `ulps` units in the last place."""
    a = got.cpu().view(torch.int16).to(torch.int32)
    b = ref.cpu().view(torch.int16).to(torch.int32)
    # map sign-magnitude to a monotone integer line
    a = torch.where(a < 0, -(a & 0x7FFF), a)
    b = torch.where(b < 0, -(b & 0x7FFF), b)
    return ((a - b).abs() > ulps).float().mean().item()


def check_sampler_picks(tokens, logits, temps, noise, what):
    """tokens must be the row-wise argmax of the oracle's scores computed from the stored logits, up to ties inside
    one bf16 ulp of a logit (the two GEMM launches may round a split tile's sum differently)."""
    from oracle import tp_path as O
    z = O.sampler_scores(logits.cpu(), temps.cpu() if temps is not None else None, noise)
    best = z.max(-1).values
    picked = z.gather(1, tokens.cpu().view(-1, 1)).squeeze(1)
    lg = logits.float().cpu().double()
    inv_t = 1.0 if temps is None else (1.0 / temps.cpu().double())
    slack = 2.0 ** -7 * (lg.abs().max(-1).values) * inv_t + 1e-4
    assert (picked >= best - slack).all(), f"{what}: a pick is below the best score by {(best - picked).max().item():.4f}"
    exact = (tokens.cpu() == z.argmax(-1)).float().mean().item()
    assert exact >= 0.9, f"{what}: only {exact * 100:.0f}% of the rows pick the oracle's token"
