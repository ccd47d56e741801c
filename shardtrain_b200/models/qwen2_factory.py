"""Build the Qwen2 module tree on the meta device.

No dense weights are allocated: registration with the sharded runtime generates (or reads from a
checkpoint) one parameter at a time and keeps only this rank's shard
(`src/sharded_runtime/models/qwen2_factory.py:8-31`).
"""

from __future__ import annotations

import torch

from shardtrain_b200.models.qwen2 import Qwen2CausalLM, Qwen2ModelConfig


def qwen_config_from(model_config) -> Qwen2ModelConfig:
    if model_config.hf_config_path:
        cfg = Qwen2ModelConfig.from_file(model_config.hf_config_path)
    else:
        cfg = Qwen2ModelConfig(
            vocab_size=model_config.vocab_size,
            hidden_size=model_config.hidden_size,
            intermediate_size=model_config.mlp_hidden_size,
            num_hidden_layers=model_config.layers,
            num_attention_heads=model_config.num_heads,
            num_key_value_heads=model_config.num_key_value_heads,
            rms_norm_eps=model_config.rms_norm_eps,
            rope_theta=model_config.rope_theta,
            tie_word_embeddings=model_config.tie_word_embeddings,
        )
    cfg.use_cache = False
    return cfg


def build_qwen_model(model_config, seed: int = 1234, *, checkpoint=None) -> Qwen2CausalLM:
    model = Qwen2CausalLM(qwen_config_from(model_config), device="meta", dtype=torch.float32)
    model._qwen_seed = seed
    path = checkpoint or model_config.checkpoint_path
    if path:
        from shardtrain_b200.models.qwen2_checkpoint import QwenCheckpoint

        model._qwen_weight_source = QwenCheckpoint(path)
    return model
