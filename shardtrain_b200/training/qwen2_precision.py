"""Compute precision of the Qwen trainer.  Master shards, gradients, communication and optimizer
state are always FP32; this only names the GEMM/activation dtype
(`src/sharded_runtime/training/qwen2_precision.py:6-20`)."""

import torch

_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


def resolve_qwen_compute_dtype(name: str, device) -> torch.dtype:
    device = torch.device(device)
    if name not in _DTYPES:
        raise ValueError("Qwen training dtype must be fp32, fp16 or bf16")
    if name == "fp16" and device.type != "cuda":
        raise ValueError("Qwen fp16 AMP requires CUDA")
    if name == "bf16" and device.type == "cuda":
        with torch.cuda.device(device):
            if not torch.cuda.is_bf16_supported(including_emulation=False):
                raise ValueError("Qwen bf16 requires native CUDA BF16 support")
    return _DTYPES[name]
