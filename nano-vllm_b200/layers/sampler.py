"""Token sampling on rank 0 (nanovllm/layers/sampler.py:5-12): temperature
softmax divided by Exp(1) noise, argmax.  Greedy decoding (temperature -> 0)
uses the library's argmax kernel directly."""
import torch
from torch import nn

from .. import ops


class Sampler(nn.Module):

    def forward(self, logits: torch.Tensor, temperatures: torch.Tensor):
        scaled = logits.float().div_(temperatures.unsqueeze(dim=1))
        probs = torch.softmax(scaled, dim=-1)
        noise = torch.empty_like(probs).exponential_(1).clamp_min_(1e-10)
        return probs.div_(noise).argmax(dim=-1)

    @staticmethod
    def greedy(logits: torch.Tensor) -> torch.Tensor:
        return ops.argmax(logits)
