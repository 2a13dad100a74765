"""Helpers shared by the GPU tests."""
import os

import numpy as np
import torch
import torch.distributed as dist

TOL_ABS, TOL_REL = 2e-2, 1e-2  # the bf16 tolerance of the path, per element: |got - ref| <= 2e-2 + 1e-2 * |ref| against an fp32 reference


def ensure_group():
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        dist.init_process_group("gloo", rank=0, world_size=1)


def error_stats(got: torch.Tensor, ref_fp32: torch.Tensor) -> dict:
    """max |err|, max |err| / |ref| over the elements with |ref| >= 1, and the worst ratio err / (abs + rel |ref|)."""
    got, ref = got.float().cpu(), ref_fp32.float().cpu()
    err = (got - ref).abs()
    big = ref.abs() >= 1.0
    return {"max_abs_err": err.max().item() if err.numel() else 0.0,
            "max_rel_err": (err[big] / ref.abs()[big]).max().item() if big.any() else 0.0,
            "worst_vs_bound": (err / (TOL_ABS + TOL_REL * ref.abs())).max().item() if err.numel() else 0.0}


def assert_close_bf16(got: torch.Tensor, ref_fp32: torch.Tensor, what: str = "", abs_tol=TOL_ABS, rel_tol=TOL_REL):
    """Every element within abs_tol + rel_tol * |its own reference value|."""
    got = got.float().cpu()
    ref = ref_fp32.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    if ref.numel() == 0:
        return
    err = (got - ref).abs()
    bound = abs_tol + rel_tol * ref.abs()
    over = err > bound
    if over.any() or not torch.isfinite(got).all():
        excess = torch.where(torch.isfinite(err), err - bound, torch.full_like(err, float("inf")))
        idx = np.unravel_index(int(excess.argmax()), err.shape)
        raise AssertionError(f"{what}: |err| {err[idx].item():.4e} > {bound[idx].item():.4e} at {idx} (got {got[idx].item():.5f}, ref {ref[idx].item():.5f}); "
                             f"{over.float().mean().item() * 100:.3f}% of elements out of tolerance; max abs err {err.max().item():.4e}")


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
