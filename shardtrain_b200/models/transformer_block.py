"""Small FP32 pre-norm decoder block (no biases, multi-head attention, SwiGLU) used by the
lifecycle tests and by the legacy TP/SP path.

The parameter names are the fixture's contract (they are what the reference toy block exposes,
`src/sharded_runtime/models/transformer_block.py:12-79`): `attention_norm.weight`,
`attention.{q,k,v,out}_proj.weight`, `mlp_norm.weight`, `mlp.{up,gate,down}_proj.weight`.  The
math is written once as functions over tensors (`rms_normalize`, `causal_attention_heads`,
`gated_mlp`); the modules only own parameters and decide whether their column projections run
one by one or through a shared-input `projection_group` installed by the TP/SP plan.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn
from torch.nn import functional as F

from shardtrain_b200.config import ModelConfig


# ---------------------------------------------------------------------------- tensor math
def rms_normalize(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + eps) * weight


def causal_attention_heads(q: Tensor, k: Tensor, v: Tensor, head_dim: int) -> Tensor:
    """Causal softmax attention of packed projections [B, S, heads * head_dim] -> same shape."""
    batch, seq, width = q.shape
    q, k, v = (t.unflatten(-1, (-1, head_dim)).transpose(1, 2) for t in (q, k, v))   # [B, h, S, d]
    scores = torch.einsum("bhqd,bhkd->bhqk", q, k) * head_dim ** -0.5
    visible = torch.ones(seq, seq, dtype=torch.bool, device=q.device).tril()
    weights = scores.masked_fill(~visible, float("-inf")).softmax(dim=-1)
    return torch.einsum("bhqk,bhkd->bqhd", weights, v).reshape(batch, seq, width)


def gated_mlp(gate: Tensor, up: Tensor) -> Tensor:
    return F.silu(gate) * up


def _linear(fan_in: int, fan_out: int) -> nn.Linear:
    return nn.Linear(fan_in, fan_out, bias=False)


# ---------------------------------------------------------------------------- parameter owners
class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float) -> None:
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(hidden_size)), eps

    def forward(self, x: Tensor) -> Tensor:
        return rms_normalize(x, self.weight, self.eps)


class _ColumnRowPair(nn.Module):
    """A sub-block whose input feeds several column projections and whose result goes through
    one row projection.  `column_names` are evaluated one by one unless a `projection_group`
    attribute was installed (one gathered input for all of them)."""

    column_names: tuple[str, ...] = ()

    def columns(self, x: Tensor):
        group = getattr(self, "projection_group", None)
        if group is not None:
            return group(x)
        return [getattr(self, name)(x) for name in self.column_names]


class CausalSelfAttention(_ColumnRowPair):
    column_names = ("q_proj", "k_proj", "v_proj")

    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        width = config.hidden_size
        self.num_heads, self.head_dim = config.num_heads, width // config.num_heads
        for name in (*self.column_names, "out_proj"):
            setattr(self, name, _linear(width, width))

    def forward(self, x: Tensor) -> Tensor:
        q, k, v = self.columns(x)
        return self.out_proj(causal_attention_heads(q, k, v, self.head_dim))


class SwiGLU(_ColumnRowPair):
    column_names = ("gate_proj", "up_proj")

    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        width, inner = config.hidden_size, config.mlp_hidden_size
        # registration order is part of the fixture: up, gate, down
        self.up_proj, self.gate_proj = _linear(width, inner), _linear(width, inner)
        self.down_proj = _linear(inner, width)

    def forward(self, x: Tensor) -> Tensor:
        gate, up = self.columns(x)
        return self.down_proj(gated_mlp(gate, up))


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
        for norm, mixer in ((self.attention_norm, self.attention), (self.mlp_norm, self.mlp)):
            x = x + mixer(norm(x))
        return x
