"""Seeded construction of the toy reference model and deterministic activation batches
(`src/sharded_runtime/models/reference.py:10-24`)."""

from __future__ import annotations

import torch
from torch import Tensor, nn

from shardtrain_b200.config import ModelConfig
from shardtrain_b200.models.transformer_block import TransformerBlock


def build_reference_model(config: ModelConfig, seed: int = 1234) -> nn.Module:
    """`nn.Sequential` of `config.layers` blocks, initialised on CPU without touching the
    caller's RNG state."""
    with torch.random.fork_rng(devices=[]):
        torch.random.default_generator.manual_seed(seed)
        return nn.Sequential(*(TransformerBlock(config) for _ in range(config.layers)))


def synthetic_batch(config: ModelConfig, batch_size: int, seed: int, *, device="cpu") -> Tensor:
    gen = torch.Generator(device="cpu").manual_seed(seed)
    shape = (batch_size, config.seq_len, config.hidden_size)
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(device)
