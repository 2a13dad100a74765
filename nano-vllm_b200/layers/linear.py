"""Tensor-parallel linear layers on the B200 GEMM kernels.

Class names, constructor signatures, parameter names and `weight_loader`
contracts are those of nanovllm/layers/linear.py (ReplicatedLinear :37,
ColumnParallelLinear :54, MergedColumnParallelLinear :76, QKVParallelLinear
:96, RowParallelLinear :131), so the reference's model code and checkpoint
loader (nanovllm/utils/loader.py:12-28) work with them unchanged.  What
differs is underneath: `forward` calls the tcgen05 GEMM through the C ABI,
and RowParallelLinear has no NCCL call: its GEMM pushes partial tiles to the
peer GPUs and finishes the reduction (and, through `forward_fused`, the
residual add and the next RMSNorm) in the same kernel launch.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from .. import ops


def divide(numerator: int, denominator: int) -> int:
    q, r = divmod(numerator, denominator)
    if r:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")
    return q


def _tp_rank_world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class LinearBase(nn.Module):
    """weight [out, in] (K contiguous), optional bias [out]; `tp_dim` is the
    dimension the loader shards (0 = output rows, 1 = input columns)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False, tp_dim: int | None = None):
        super().__init__()
        self.tp_dim = tp_dim
        self.tp_rank, self.tp_size = _tp_rank_world()
        self.weight = nn.Parameter(torch.empty(output_size, input_size), requires_grad=False)
        self.weight.weight_loader = self.weight_loader
        if bias:
            self.bias = nn.Parameter(torch.empty(output_size), requires_grad=False)
            self.bias.weight_loader = self.weight_loader
        else:
            self.register_parameter("bias", None)

    def _shard_of(self, full: torch.Tensor, dim: int) -> torch.Tensor:
        return full.chunk(self.tp_size, dim)[self.tp_rank]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class ReplicatedLinear(LinearBase):

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        super().__init__(input_size, output_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(loaded_weight)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.gemm(x, self.weight, self.bias)


class ColumnParallelLinear(LinearBase):
    """Output features split over ranks; no communication."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        _, world = _tp_rank_world()
        super().__init__(input_size, divide(output_size, world), bias, 0)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        param.data.copy_(self._shard_of(loaded_weight, self.tp_dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.gemm(x, self.weight, self.bias)


class MergedColumnParallelLinear(ColumnParallelLinear):
    """Several column-parallel matrices stacked along the output dimension
    (gate_proj and up_proj).  Shard `i` of a checkpoint tensor lands at row
    offset sum(output_sizes[:i]) / tp_size of the local weight.

    `pair_rows()` (before loading) switches the stored layout to the one the
    fused gate_up + SiLU*mul GEMM reads: the two matrices' rows interleaved
    (row 2j = first matrix's row j, row 2j+1 = second matrix's row j).  The
    loader then writes each shard straight into its rows, so no second copy of
    the weight exists; `forward` still returns [first | second] columns."""

    def __init__(self, input_size: int, output_sizes: list[int], bias: bool = False):
        self.output_sizes = list(output_sizes)
        self.paired = False
        super().__init__(input_size, sum(output_sizes), bias)

    def pair_rows(self) -> "MergedColumnParallelLinear":
        assert len(self.output_sizes) == 2 and self.output_sizes[0] == self.output_sizes[1] and self.bias is None
        self.paired = True
        self._pairs = None
        return self

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: int):
        shard = self._shard_of(loaded_weight, self.tp_dim)
        if self.paired:
            param.data[loaded_shard_id::2].copy_(shard)
        else:
            offset = sum(self.output_sizes[:loaded_shard_id]) // self.tp_size
            size = self.output_sizes[loaded_shard_id] // self.tp_size
            param.data.narrow(self.tp_dim, offset, size).copy_(shard)
        self._pairs = None

    _pairs: torch.Tensor | None = None

    def paired_weight(self) -> torch.Tensor:
        """The local weight with the two halves' rows interleaved: the layout ops.gemm_silu_mul reads.  With
        pair_rows() it is `weight` itself; otherwise a second copy built once from the reference's
        [first half ; second half] layout the first time it is asked for."""
        if self.paired:
            return self.weight.data
        if self._pairs is None:
            assert len(self.output_sizes) == 2 and self.output_sizes[0] == self.output_sizes[1] and self.bias is None
            half = self.weight.shape[0] // 2
            w = self.weight.data
            self._pairs = torch.stack((w[:half], w[half:]), dim=1).reshape(2 * half, w.shape[1]).contiguous()
        return self._pairs

    def reference_weight(self) -> torch.Tensor:
        """The local weight in the reference's layout [first half ; second half] (a copy when the rows are paired)."""
        if not self.paired:
            return self.weight.data
        return torch.cat((self.weight.data[0::2], self.weight.data[1::2]), dim=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.gemm(x, self.weight, self.bias)
        if self.paired:  # columns come out as (first_0, second_0, first_1, ...): back to [first | second]
            y = torch.cat((y[..., 0::2], y[..., 1::2]), dim=-1)
        return y

    def forward_silu_mul(self, x: torch.Tensor) -> torch.Tensor:
        """SiLU(first half) * second half of forward(x), in the GEMM's epilogue."""
        return ops.gemm_silu_mul(x, self.paired_weight())


class QKVParallelLinear(ColumnParallelLinear):
    """Local rows are [this rank's q heads ; its k heads ; its v heads]."""

    def __init__(self, hidden_size: int, head_size: int, total_num_heads: int, total_num_kv_heads: int | None = None, bias: bool = False):
        _, world = _tp_rank_world()
        total_num_kv_heads = total_num_kv_heads or total_num_heads
        self.head_size = head_size
        self.num_heads = divide(total_num_heads, world)
        self.num_kv_heads = divide(total_num_kv_heads, world)
        super().__init__(hidden_size, (total_num_heads + 2 * total_num_kv_heads) * head_size, bias)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor, loaded_shard_id: str):
        q_rows, kv_rows = self.num_heads * self.head_size, self.num_kv_heads * self.head_size
        layout = {"q": (0, q_rows), "k": (q_rows, kv_rows), "v": (q_rows + kv_rows, kv_rows)}
        assert loaded_shard_id in layout
        offset, size = layout[loaded_shard_id]
        param.data.narrow(self.tp_dim, offset, size).copy_(self._shard_of(loaded_weight, self.tp_dim))


class RowParallelLinear(LinearBase):
    """Input features split over ranks; the partial products are summed over
    ranks.  `forward(x)` keeps the reference's meaning (returns the summed y).
    `forward_fused(x, residual, norm)` additionally applies the RMSNorm that
    follows in the decoder layer and returns (normed, new_residual), all in one
    kernel launch per rank."""

    def __init__(self, input_size: int, output_size: int, bias: bool = False):
        _, world = _tp_rank_world()
        super().__init__(divide(input_size, world), output_size, bias, 1)

    def weight_loader(self, param: nn.Parameter, loaded_weight: torch.Tensor):
        if param.data.ndim == 1:  # the bias is not sharded
            param.data.copy_(loaded_weight)
        else:
            param.data.copy_(self._shard_of(loaded_weight, self.tp_dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rowpar_fused(x, self.weight, self.bias, None, None, 0.0)

    def forward_fused(self, x: torch.Tensor, residual: torch.Tensor, norm) -> tuple[torch.Tensor, torch.Tensor]:
        return ops.rowpar_fused(x, self.weight, self.bias, residual, norm.weight, norm.eps)
