"""Dense Qwen2 / Qwen2.5 decoder with Hugging Face parameter names.

This is the unsharded form of the model: the oracle for tests, the CPU path, and the module
skeleton whose parameters the sharded runtime replaces with flat FP32 shards.  The equations are
the public Qwen2 architecture: pre-norm residual blocks, RMSNorm with FP32 accumulation, rotary
embedding in `rotate_half` form from *global* positions, grouped-query causal attention with an
optional `[B, S]` key-padding mask (a fully masked query row yields zeros), SwiGLU MLP, optional
tied LM head.  Parameter names, config fields and rejections follow
`src/sharded_runtime/models/qwen2.py:22-417`; the math lives in free functions (`rms_norm`,
`rotary_tables`, `apply_rotary`, `causal_attention`, `swiglu`) so the sharded executors can call
the same code with materialised weights.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

import torch
import yaml
from torch import Tensor, nn
from torch.nn import functional as F


@dataclass
class Qwen2ModelConfig:
    vocab_size: int = 128
    hidden_size: int = 32
    intermediate_size: int = 64
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    initializer_range: float = 0.02
    attention_dropout: float = 0.0
    tie_word_embeddings: bool = True
    hidden_act: str = "silu"
    pad_token_id: int | None = None
    bos_token_id: int | None = None
    eos_token_id: int | list[int] | None = None
    use_cache: bool = False
    use_sliding_window: bool = False
    model_type: str = "qwen2"
    rope_scaling: dict[str, Any] | None = None

    def __post_init__(self) -> None:
        dims = {
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "max_position_embeddings": self.max_position_embeddings,
        }
        if any(v <= 0 for v in dims.values()):
            raise ValueError("Qwen2 dimensions must be positive")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2:
            raise ValueError("Qwen2 RoPE requires an even head dimension")
        if self.model_type != "qwen2" or self.hidden_act != "silu":
            raise ValueError("Only the Qwen2 decoder with SiLU SwiGLU is supported")
        if self.use_sliding_window:
            raise ValueError("Sliding-window attention is outside this training adapter's scope")
        if self.rope_scaling is not None:
            raise ValueError("RoPE scaling/YaRN is outside this training adapter's scope")
        if self.rope_theta <= 0 or self.rms_norm_eps <= 0:
            raise ValueError("rope_theta and rms_norm_eps must be positive")
        if not 0 <= self.attention_dropout < 1:
            raise ValueError("attention_dropout must be in [0, 1)")
        if self.pad_token_id is not None and not 0 <= self.pad_token_id < self.vocab_size:
            raise ValueError("pad_token_id is outside the vocabulary")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_dict(cls, values: dict[str, Any]) -> "Qwen2ModelConfig":
        if not isinstance(values, dict):
            raise ValueError("Qwen2 configuration must be a mapping")
        # HF files also carry serialisation / inference metadata that is not part of the model.
        kept = {k: v for k, v in values.items() if k in cls.__dataclass_fields__}
        if kept.get("num_key_value_heads") is None:
            kept["num_key_value_heads"] = kept.get("num_attention_heads", 4)
        rope = values.get("rope_parameters")
        if rope:
            if rope.get("rope_type", "default") != "default":
                raise ValueError("Only default Qwen2 RoPE is supported")
            kept["rope_theta"] = rope.get("rope_theta", 1000000.0)
        natural = kept.get("hidden_size", 32) // kept.get("num_attention_heads", 4)
        if values.get("head_dim", natural) != natural:
            raise ValueError("A custom head_dim is unsupported for Qwen2.5")
        kinds = values.get("layer_types")
        if kinds is not None and any(kind != "full_attention" for kind in kinds):
            raise ValueError("Only full causal attention layers are supported")
        return cls(**kept)

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen2ModelConfig":
        return cls.from_dict(json.loads(Path(path).read_text(encoding="utf-8")))

    @classmethod
    def from_file(cls, path: str | Path) -> "Qwen2ModelConfig":
        path = Path(path)
        suffix = path.suffix.lower()
        if suffix == ".json":
            return cls.from_json(path)
        if suffix in {".yaml", ".yml"}:
            return cls.from_dict(yaml.safe_load(path.read_text(encoding="utf-8")))
        raise ValueError("Qwen2 configuration must use .yaml, .yml or .json")

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


# ---------------------------------------------------------------------------- functional math
def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """FP32 accumulation; the normalised value is rounded to x's dtype before the scale."""
    wide = x.float()
    scale = torch.rsqrt(wide.square().mean(dim=-1, keepdim=True) + eps)
    return weight * (wide * scale).to(x.dtype)


def rotary_inverse_frequencies(head_dim: int, theta: float, device=None) -> Tensor:
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
    return theta ** (-exponent)


def rotary_tables(position_ids: Tensor, inv_freq: Tensor, dtype: torch.dtype) -> tuple[Tensor, Tensor]:
    """cos/sin of shape [B or 1, S, head_dim] computed in FP32 from global positions."""
    with torch.autocast(device_type=position_ids.device.type, enabled=False):
        angle = position_ids.float().unsqueeze(-1) * inv_freq.float()
        angle = torch.cat((angle, angle), dim=-1)
        return angle.cos().to(dtype), angle.sin().to(dtype)


def rotate_half(x: Tensor) -> Tensor:
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


def apply_rotary(q: Tensor, k: Tensor, cos: Tensor, sin: Tensor) -> tuple[Tensor, Tensor]:
    """q, k: [B, heads, S, D]; cos, sin: [B or 1, S, D]."""
    cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def _with_key_padding(lower: Tensor, mask: Tensor, like: Tensor) -> Tensor:
    """[B, S] key mask: a key is visible when it is causal AND not padding."""
    batch, seq = like.shape[0], like.shape[2]
    if mask.shape != (batch, seq):
        raise ValueError("attention_mask must describe the full global [batch, sequence]")
    return lower & mask.bool()[:, None, None, :]


def _with_full_mask(lower: Tensor, mask: Tensor, like: Tensor) -> Tensor:
    """[B or 1, 1, S, S] mask: boolean masks are intersected with the causal triangle, additive
    floating-point masks get the triangle's complement filled with the dtype's minimum."""
    batch, seq = like.shape[0], like.shape[2]
    if mask.shape[-2:] != (seq, seq):
        raise ValueError("attention_mask must have shape [B,S] or [B,1,S,S]")
    if mask.shape[0] not in (1, batch):
        raise ValueError("attention_mask batch size is incompatible")
    if mask.dtype == torch.bool:
        return lower & mask
    if not mask.is_floating_point():
        raise ValueError("A 4-D attention mask must be boolean or additive floating point")
    return mask.to(like.dtype).masked_fill(~lower, torch.finfo(like.dtype).min)


_MASK_FORMS = {2: _with_key_padding, 4: _with_full_mask}      # by number of dimensions


def causal_attention_mask(x: Tensor, attention_mask: Tensor | None) -> Tensor:
    """Boolean (or additive, for a float 4-D input) mask for [B, H, S, D] queries."""
    batch, _, seq, _ = x.shape
    lower = torch.ones((seq, seq), dtype=torch.bool, device=x.device).tril()
    lower = lower[None, None].expand(batch, 1, seq, seq)
    if attention_mask is None:
        return lower
    combine = _MASK_FORMS.get(attention_mask.ndim)
    if combine is None:
        raise ValueError("attention_mask must have shape [B,S] or [B,1,S,S]")
    return combine(lower, attention_mask.to(x.device), x)


def causal_attention(q: Tensor, k: Tensor, v: Tensor, attention_mask: Tensor | None) -> Tensor:
    """Grouped-query causal attention.  q: [B, Hq, S, D]; k, v: [B, Hkv, S, D] -> [B, Hq, S, D].

    Scores and softmax are FP32; rows with no allowed key produce zeros.
    """
    groups = q.shape[1] // k.shape[1]
    if groups > 1:
        k, v = k.repeat_interleave(groups, dim=1), v.repeat_interleave(groups, dim=1)
    mask = causal_attention_mask(q, attention_mask)
    scores = torch.matmul(q, k.transpose(-1, -2)).float() / math.sqrt(q.shape[-1])
    if mask.dtype == torch.bool:
        scores = scores.masked_fill(~mask, float("-inf"))
        dead = ~mask.any(dim=-1, keepdim=True)
        probs = torch.softmax(scores.masked_fill(dead, 0.0), dim=-1).masked_fill(dead, 0.0)
    else:
        probs = torch.softmax(scores + mask.float(), dim=-1)
    return torch.matmul(probs.to(v.dtype), v)


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return F.silu(gate) * up


def causal_lm_loss_parts(logits: Tensor, labels: Tensor) -> tuple[Tensor, Tensor]:
    """(FP32 sum of next-token losses, number of valid labels); no mean of local means."""
    if logits.ndim != 3 or labels.shape != logits.shape[:2]:
        raise ValueError("labels must match the complete logits [batch, sequence]")
    target = labels[:, 1:].contiguous()
    count = target.ne(-100).sum()
    if target.numel() == 0:
        return logits.float().sum() * 0.0, count
    total = F.cross_entropy(
        logits[:, :-1].float().reshape(-1, logits.shape[-1]),
        target.reshape(-1),
        ignore_index=-100,
        reduction="sum",
    )
    return total, count


# ---------------------------------------------------------------------------- modules
class Qwen2RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, **factory: Any) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, **factory))
        self.eps = self.variance_epsilon = eps

    def forward(self, x: Tensor) -> Tensor:
        return rms_norm(x, self.weight, self.eps)


class Qwen2RotaryEmbedding(nn.Module):
    def __init__(self, config: Qwen2ModelConfig, device: Any = None) -> None:
        super().__init__()
        inv = rotary_inverse_frequencies(config.head_dim, config.rope_theta, device)
        self.register_buffer("inv_freq", inv, persistent=False)

    def forward(self, x: Tensor, position_ids: Tensor) -> tuple[Tensor, Tensor]:
        return rotary_tables(position_ids, self.inv_freq, x.dtype)


class Qwen2Attention(nn.Module):
    def __init__(self, config: Qwen2ModelConfig, layer_idx: int, **factory: Any) -> None:
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.head_dim
        h, d = config.hidden_size, config.head_dim
        self.q_proj = nn.Linear(h, self.num_heads * d, bias=True, **factory)
        self.k_proj = nn.Linear(h, self.num_key_value_heads * d, bias=True, **factory)
        self.v_proj = nn.Linear(h, self.num_key_value_heads * d, bias=True, **factory)
        self.o_proj = nn.Linear(self.num_heads * d, h, bias=False, **factory)
        self.position_embeddings: tuple[Tensor, Tensor] | None = None
        self.attention_mask: Tensor | None = None

    def forward(self, x: Tensor) -> Tensor:
        if self.position_embeddings is None:
            raise RuntimeError("Qwen2Attention requires the full-sequence position context")
        batch, seq, _ = x.shape

        def heads(t: Tensor, n: int) -> Tensor:
            return t.reshape(batch, seq, n, self.head_dim).transpose(1, 2)

        q = heads(self.q_proj(x), self.num_heads)
        k = heads(self.k_proj(x), self.num_key_value_heads)
        v = heads(self.v_proj(x), self.num_key_value_heads)
        cos, sin = self.position_embeddings
        if cos.shape[-2] != seq:
            raise ValueError("QKV sequence length differs from global RoPE positions")
        q, k = apply_rotary(q, k, cos, sin)
        mixed = causal_attention(q, k, v, self.attention_mask)
        return self.o_proj(mixed.transpose(1, 2).reshape(batch, seq, -1))


class Qwen2MLP(nn.Module):
    def __init__(self, config: Qwen2ModelConfig, **factory: Any) -> None:
        super().__init__()
        h, i = config.hidden_size, config.intermediate_size
        self.gate_proj = nn.Linear(h, i, bias=False, **factory)
        self.up_proj = nn.Linear(h, i, bias=False, **factory)
        self.down_proj = nn.Linear(i, h, bias=False, **factory)

    def forward(self, x: Tensor) -> Tensor:
        return self.down_proj(swiglu(self.gate_proj(x), self.up_proj(x)))


class Qwen2DecoderLayer(nn.Module):
    def __init__(self, config: Qwen2ModelConfig, layer_idx: int, **factory: Any) -> None:
        super().__init__()
        self.hidden_size = config.hidden_size
        self.self_attn = Qwen2Attention(config, layer_idx, **factory)
        self.mlp = Qwen2MLP(config, **factory)
        self.input_layernorm = Qwen2RMSNorm(config.hidden_size, config.rms_norm_eps, **factory)
        self.post_attention_layernorm = Qwen2RMSNorm(config.hidden_size, config.rms_norm_eps, **factory)

    def forward(self, x: Tensor) -> Tensor:
        x = x + self.self_attn(self.input_layernorm(x))
        return x + self.mlp(self.post_attention_layernorm(x))


class Qwen2Model(nn.Module):
    def __init__(self, config: Qwen2ModelConfig, **factory: Any) -> None:
        super().__init__()
        self.embed_tokens = nn.Embedding(
            config.vocab_size, config.hidden_size, padding_idx=config.pad_token_id, **factory
        )
        self.layers = nn.ModuleList(
            Qwen2DecoderLayer(config, i, **factory) for i in range(config.num_hidden_layers)
        )
        self.norm = Qwen2RMSNorm(config.hidden_size, config.rms_norm_eps, **factory)
        self.rotary_emb = Qwen2RotaryEmbedding(config, device=factory.get("device"))


@dataclass
class Qwen2CausalLMOutput:
    logits: Tensor | None
    loss: Tensor | None = None
    last_hidden_state: Tensor | None = None


class Qwen2CausalLM(nn.Module):
    def __init__(self, config: Qwen2ModelConfig | Any, *, device: Any = None,
                 dtype: torch.dtype | None = None) -> None:
        super().__init__()
        if not isinstance(config, Qwen2ModelConfig):
            config = Qwen2ModelConfig.from_dict(config.to_dict())
        self.config = config
        self.model = Qwen2Model(config, device=device, dtype=dtype)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False, device=device, dtype=dtype)
        self.apply(self._init_weights)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def _init_weights(self, module: nn.Module) -> None:
        if isinstance(module, (nn.Linear, nn.Embedding)):
            if module.weight.device.type == "meta":
                return
            nn.init.normal_(module.weight, mean=0.0, std=self.config.initializer_range)
            if isinstance(module, nn.Linear) and module.bias is not None:
                nn.init.zeros_(module.bias)
            if isinstance(module, nn.Embedding) and module.padding_idx is not None:
                with torch.no_grad():
                    module.weight[module.padding_idx].zero_()

    def forward(self, input_ids: Tensor | None = None, attention_mask: Tensor | None = None,
                position_ids: Tensor | None = None, labels: Tensor | None = None,
                inputs_embeds: Tensor | None = None, use_cache: bool = False) -> Qwen2CausalLMOutput:
        if use_cache:
            raise ValueError("This adapter supports training with use_cache=False only")
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("Specify exactly one of input_ids or inputs_embeds")
        source = input_ids if input_ids is not None else inputs_embeds
        batch, seq = source.shape[:2]
        default_positions = position_ids is None
        if position_ids is None:
            position_ids = torch.arange(seq, device=source.device).unsqueeze(0)
        if tuple(position_ids.shape) not in ((1, seq), (batch, seq)):
            raise ValueError("position_ids must describe the complete global sequence")
        if inputs_embeds is not None and inputs_embeds.shape[-1] != self.config.hidden_size:
            raise ValueError("inputs_embeds hidden size differs from config.hidden_size")
        runtime = getattr(self, "_sharded_runtime", None)
        if runtime is not None:
            # The sharded runtime owns the step: it walks its units with materialised weights.
            return runtime.model_forward(
                self, input_ids, attention_mask=attention_mask, position_ids=position_ids,
                labels=labels, inputs_embeds=inputs_embeds, default_positions=default_positions,
            )
        hidden = self.model.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        tables = self.model.rotary_emb(hidden, position_ids.to(hidden.device))
        for index, layer in enumerate(self.model.layers):
            layer.self_attn.position_embeddings = tables
            layer.self_attn.attention_mask = attention_mask
            with torch.profiler.record_function(f"shardtrain/qwen/layer{index}"):
                hidden = layer(hidden)
        hidden = self.model.norm(hidden)
        logits = self.lm_head(hidden)
        loss = None
        if labels is not None:
            total, count = causal_lm_loss_parts(logits, labels)
            loss = total / count.clamp_min(1)
        return Qwen2CausalLMOutput(logits=logits, loss=loss, last_hidden_state=hidden)


Qwen2Config = Qwen2ModelConfig
Qwen2ForCausalLM = Qwen2CausalLM
