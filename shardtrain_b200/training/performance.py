"""Architecture FLOP accounting shared by every engine that is compared
(`src/sharded_runtime/training/performance.py:6-57`): 6 * N * tokens for the dense layers plus
12 * L * H * S * tokens for attention.  MFU is reported only against a peak the caller supplies."""

from __future__ import annotations

import math


def model_flops_per_step(parameter_numel, layers, hidden_size, sequence_length, global_batch):
    tokens = global_batch * sequence_length
    dense = 6 * parameter_numel * tokens
    attention = 12 * layers * hidden_size * sequence_length * tokens
    return tokens, dense, attention


def qwen_performance_summary(*, parameter_numel, layers, hidden_size, sequence_length, global_batch,
                             steps, world_size, peak_tflops_per_gpu=None, profile_mode="off"):
    if peak_tflops_per_gpu is not None and (
            not math.isfinite(peak_tflops_per_gpu) or peak_tflops_per_gpu <= 0):
        raise ValueError("peak_tflops_per_gpu must be a finite positive nominal peak")
    tokens, dense, attention = model_flops_per_step(parameter_numel, layers, hidden_size,
                                                    sequence_length, global_batch)
    durations = [row["max_rank_seconds"] for row in steps]
    if any(not math.isfinite(t) or t <= 0 for t in durations):
        raise ValueError("Measured max-rank step durations must be finite and positive")
    elapsed = sum(durations)
    mean = elapsed / len(durations) if durations else None
    tflops = (dense + attention) / mean / 1e12 if mean else None
    mfu = None
    if tflops is not None and peak_tflops_per_gpu is not None:
        mfu = 100 * tflops / (world_size * peak_tflops_per_gpu)
    per_second = (lambda amount: amount / elapsed) if elapsed else (lambda amount: None)
    return {
        "flops_formula": "6 * unique_parameters * input_tokens + "
                         "12 * layers * hidden_size * sequence * input_tokens",
        "model_unique_parameters": parameter_numel,
        "global_input_tokens_per_step": tokens,
        "six_n_flops_per_step": dense,
        "attention_flops_per_step": attention,
        "estimated_model_flops_per_step": dense + attention,
        "mean_max_rank_seconds": mean,
        "global_input_tokens_per_second": per_second(tokens * len(durations)),
        "global_valid_tokens_per_second": per_second(sum(row["valid_tokens"] for row in steps)),
        "global_sequences_per_second": per_second(global_batch * len(durations)),
        "all_gpu_effective_model_tflops": tflops,
        "peak_tflops_per_gpu": peak_tflops_per_gpu,
        "mfu_percent": mfu,
        "profile_mode": profile_mode,
        "unprofiled_timing": profile_mode == "off",
        "limitations": "architecture estimate over input positions; excludes optimizer, "
                       "elementwise work and communication; peak must be supplied explicitly",
    }
