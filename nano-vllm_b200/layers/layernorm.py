"""RMSNorm on hand-written CUDA kernels (no torch.compile, no Triton).

Same interface as nanovllm/layers/layernorm.py:5-50: forward(x) -> normed,
forward(x, residual) -> (normed, x + residual).  Statistics are fp32; the
normalised value is rounded to bf16 before the multiplication by the weight,
and with a residual the statistics come from the un-rounded fp32 sum, as in
the reference.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


class RMSNorm(nn.Module):

    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size), requires_grad=False)

    def rms_forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_rms_forward(self, x: torch.Tensor, residual: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        return self.rms_forward(x) if residual is None else self.add_rms_forward(x, residual)
