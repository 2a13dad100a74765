"""Qwen3 decoder wired for the fused tensor-parallel path.

Module and parameter names are those of nanovllm/models/qwen3.py, so a
checkpoint (or the reference's loader, nanovllm/utils/loader.py) addresses the
same tensors.  The data flow differs in where the norms run:

  reference (:146-159)                      here
  --------------------------------------   ------------------------------------------
  h, res = input_layernorm(h, res)          (done by the previous layer's down_proj launch)
  h = attn(h)          # o_proj + NCCL      qkv GEMM with q/k-norm + RoPE + KV scatter in its epilogue;
  h, res = post_attention_layernorm(h,res)  attention (library); o_proj GEMM + cross-GPU sum
  h = mlp(h)           # down_proj + NCCL     + residual + post_attention_layernorm (1 kernel);
                                            gate_up GEMM with SiLU*mul in its epilogue; down_proj GEMM + cross-GPU
                                              sum + residual + NEXT layer's input_layernorm
                                              (or the final norm) (1 kernel)
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..layers.activation import SiluAndMul
from ..layers.attention import Attention
from ..layers.embed_head import ParallelLMHead, VocabParallelEmbedding
from ..layers.layernorm import RMSNorm
from ..layers.linear import MergedColumnParallelLinear, QKVParallelLinear, RowParallelLinear, _tp_rank_world
from ..layers.rotary_embedding import get_rope
from ..utils.context import get_context


class Qwen3Attention(nn.Module):

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, max_position: int = 4096 * 32, head_dim: int | None = None,
                 rms_norm_eps: float = 1e-06, qkv_bias: bool = False, rope_theta: float = 10000, rope_scaling: dict | None = None) -> None:
        super().__init__()
        _, tp = _tp_rank_world()
        assert num_heads % tp == 0 and num_kv_heads % tp == 0
        self.total_num_heads, self.total_num_kv_heads = num_heads, num_kv_heads
        self.num_heads, self.num_kv_heads = num_heads // tp, num_kv_heads // tp
        self.head_dim = head_dim or hidden_size // num_heads
        self.q_size, self.kv_size = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        self.scaling = self.head_dim ** -0.5
        self.qkv_bias = qkv_bias
        self.rms_norm_eps = rms_norm_eps
        self.qkv_proj = QKVParallelLinear(hidden_size, self.head_dim, num_heads, num_kv_heads, bias=qkv_bias)
        self.o_proj = RowParallelLinear(num_heads * self.head_dim, hidden_size, bias=False)
        if isinstance(rope_scaling, dict):
            rope_theta = rope_scaling.get("rope_theta", rope_theta)
        self.rotary_emb = get_rope(self.head_dim, rotary_dim=self.head_dim, max_position=max_position, base=rope_theta)
        self.attn = Attention(self.num_heads, self.head_dim, self.scaling, self.num_kv_heads)
        if not qkv_bias:
            self.q_norm = RMSNorm(self.head_dim, eps=rms_norm_eps)
            self.k_norm = RMSNorm(self.head_dim, eps=rms_norm_eps)

    def attention_output(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        """Everything up to (not including) o_proj: returns [T, q_size]."""
        ctx = get_context()
        have_cache = self.attn.k_cache.numel() > 0
        # projection, q/k head norm, RoPE and the K/V scatter: one launch for decode-sized batches, two otherwise
        qkv = ops.qkv_fused(hidden_states, self.qkv_proj.weight, self.qkv_proj.bias, self.num_heads, self.num_kv_heads, self.head_dim,
                            None if self.qkv_bias else self.q_norm.weight, None if self.qkv_bias else self.k_norm.weight,
                            self.rms_norm_eps, positions, self.rotary_emb.cos_sin_cache,
                            self.attn.k_cache if have_cache else None, self.attn.v_cache if have_cache else None,
                            ctx.slot_mapping if have_cache else None)
        q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        o = self.attn.attend(q.view(-1, self.num_heads, self.head_dim), k.view(-1, self.num_kv_heads, self.head_dim),
                             v.view(-1, self.num_kv_heads, self.head_dim))
        return o.reshape(-1, self.q_size)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.o_proj(self.attention_output(positions, hidden_states))


class Qwen3MLP(nn.Module):

    def __init__(self, hidden_size: int, intermediate_size: int, hidden_act: str) -> None:
        super().__init__()
        assert hidden_act == "silu"
        # rows stored interleaved (gate_j, up_j): the layout the fused gate_up + SiLU*mul launch reads, filled by the loader
        self.gate_up_proj = MergedColumnParallelLinear(hidden_size, [intermediate_size] * 2, bias=False).pair_rows()
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias=False)
        self.act_fn = SiluAndMul()

    def activation(self, x: torch.Tensor) -> torch.Tensor:
        """act_fn(gate_up_proj(x)) in one launch: the SiLU * mul runs in the GEMM's epilogue."""
        return self.gate_up_proj.forward_silu_mul(x)

    def forward(self, x):
        return self.down_proj(self.activation(x))


class Qwen3DecoderLayer(nn.Module):

    def __init__(self, config) -> None:
        super().__init__()
        rope_params = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None)
        self.self_attn = Qwen3Attention(
            hidden_size=config.hidden_size, num_heads=config.num_attention_heads, num_kv_heads=config.num_key_value_heads,
            max_position=config.max_position_embeddings, rms_norm_eps=config.rms_norm_eps,
            qkv_bias=getattr(config, "attention_bias", True), head_dim=getattr(config, "head_dim", None),
            rope_theta=getattr(config, "rope_theta", 1000000), rope_scaling=rope_params)
        self.mlp = Qwen3MLP(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size, hidden_act=config.hidden_act)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, positions: torch.Tensor, normed: torch.Tensor, residual: torch.Tensor, next_norm: RMSNorm):
        """`normed` is this layer's input_layernorm output, `residual` the
        residual stream that goes with it.  Returns the NEXT norm's output and
        the residual stream after this layer."""
        attn = self.self_attn.attention_output(positions, normed)
        normed, residual = self.self_attn.o_proj.forward_fused(attn, residual, self.post_attention_layernorm)
        act = self.mlp.activation(normed)
        return self.mlp.down_proj.forward_fused(act, residual, next_norm)


class Qwen3Model(nn.Module):

    def __init__(self, config) -> None:
        super().__init__()
        self.embed_tokens = VocabParallelEmbedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([Qwen3DecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        residual = self.embed_tokens(input_ids)
        # layer 0 has no residual yet: plain norm, the embedding becomes the residual (reference :152-153)
        normed = self.layers[0].input_layernorm(residual)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            next_norm = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            normed, residual = layer(positions, normed, residual, next_norm)
        return normed


class Qwen3ForCausalLM(nn.Module):
    packed_modules_mapping = {
        "q_proj": ("qkv_proj", "q"),
        "k_proj": ("qkv_proj", "k"),
        "v_proj": ("qkv_proj", "v"),
        "gate_proj": ("gate_up_proj", 0),
        "up_proj": ("gate_up_proj", 1),
    }

    def __init__(self, config) -> None:
        super().__init__()
        self.model = Qwen3Model(config)
        self.lm_head = ParallelLMHead(config.vocab_size, config.hidden_size)
        if config.tie_word_embeddings:
            self.lm_head.weight.data = self.model.embed_tokens.weight.data

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        return self.model(input_ids, positions)

    def compute_logits(self, hidden_states: torch.Tensor):
        return self.lm_head(hidden_states)

    def sample_tokens(self, hidden_states: torch.Tensor, temperatures: torch.Tensor | None, seed: int, out: torch.Tensor | None = None):
        """compute_logits + the sampler in one pass (token ids valid on rank 0); see ParallelLMHead.forward_sample."""
        return self.lm_head.forward_sample(hidden_states, temperatures, seed, out)

    def load_full_weights(self, weights: dict[str, torch.Tensor]) -> None:
        """Feed full (unsharded) tensors under HF names through every
        parameter's weight_loader, as nanovllm/utils/loader.py:12-28 does for a
        safetensors file; each rank keeps its shard."""
        for name, tensor in weights.items():
            for key, (packed, shard_id) in self.packed_modules_mapping.items():
                if key in name:
                    param = self.get_parameter(name.replace(key, packed))
                    param.weight_loader(param, tensor.to(param.device), shard_id)
                    break
            else:
                param = self.get_parameter(name)
                loader = getattr(param, "weight_loader", None)
                if loader is None:
                    param.data.copy_(tensor)
                else:
                    loader(param, tensor.to(param.device))
