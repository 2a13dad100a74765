"""SiLU(gate) * up as one CUDA kernel (nanovllm/layers/activation.py:6-11)."""
from torch import nn

from .. import ops


class SiluAndMul(nn.Module):

    def forward(self, x):
        return ops.silu_and_mul(x)
