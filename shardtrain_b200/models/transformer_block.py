"""Small FP32 pre-norm decoder block (no biases, MHA, SwiGLU) used by lifecycle tests and the
legacy TP/SP path.  Parameter names match the reference toy block
(`src/sharded_runtime/models/transformer_block.py:12-79`): `attention_norm.weight`,
`attention.{q,k,v,out}_proj.weight`, `mlp_norm.weight`, `mlp.{up,gate,down}_proj.weight`.
"""

from __future__ import annotations

import math

import torch
from torch import Tensor, nn
from torch.nn import functional as F

from shardtrain_b200.config import ModelConfig


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: Tensor) -> Tensor:
        return x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + self.eps) * self.weight


def masked_softmax_attention(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """Explicit causal softmax attention on [B, H, S, D] tensors."""
    seq = q.shape[-2]
    scores = (q @ k.transpose(-2, -1)) / math.sqrt(q.shape[-1])
    future = torch.ones((seq, seq), dtype=torch.bool, device=q.device).triu(diagonal=1)
    return scores.masked_fill(future, float("-inf")).softmax(dim=-1) @ v


class CausalSelfAttention(nn.Module):
    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        h = config.hidden_size
        self.num_heads = config.num_heads
        self.head_dim = h // config.num_heads
        self.q_proj = nn.Linear(h, h, bias=False)
        self.k_proj = nn.Linear(h, h, bias=False)
        self.v_proj = nn.Linear(h, h, bias=False)
        self.out_proj = nn.Linear(h, h, bias=False)

    def forward(self, x: Tensor) -> Tensor:
        group = getattr(self, "projection_group", None)
        parts = group(x) if group else [p(x) for p in (self.q_proj, self.k_proj, self.v_proj)]
        batch, seq, width = parts[0].shape
        q, k, v = (t.reshape(batch, seq, -1, self.head_dim).transpose(1, 2) for t in parts)
        mixed = masked_softmax_attention(q, k, v)
        return self.out_proj(mixed.transpose(1, 2).contiguous().reshape(batch, seq, width))


class SwiGLU(nn.Module):
    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        h, i = config.hidden_size, config.mlp_hidden_size
        self.up_proj = nn.Linear(h, i, bias=False)
        self.gate_proj = nn.Linear(h, i, bias=False)
        self.down_proj = nn.Linear(i, h, bias=False)

    def forward(self, x: Tensor) -> Tensor:
        group = getattr(self, "projection_group", None)
        gate, up = group(x) if group else (self.gate_proj(x), self.up_proj(x))
        return self.down_proj(F.silu(gate) * up)


class TransformerBlock(nn.Module):
    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        self.hidden_size = config.hidden_size
        self.attention_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.attention = CausalSelfAttention(config)
        self.mlp_norm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.mlp = SwiGLU(config)

    def forward(self, x: Tensor) -> Tensor:
        if x.ndim != 3 or x.shape[-1] != self.hidden_size:
            raise ValueError(f"Expected [batch, sequence, {self.hidden_size}], got {tuple(x.shape)}")
        x = x + self.attention(self.attention_norm(x))
        return x + self.mlp(self.mlp_norm(x))
