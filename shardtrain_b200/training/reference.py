"""Functional dense oracle of the toy block stack (no model code involved) and a tensor
comparison helper (`src/sharded_runtime/training/reference.py:7-65`)."""

from __future__ import annotations

import torch
from torch.nn import functional as F


def dense_oracle(x, parameters, config, *, sublayers=None):
    """Run `config.layers` blocks from a name->tensor dict; returns every block's output.
    When `sublayers` is a list, the intermediate tensors of every block are appended to it."""
    outputs = []
    heads = config.num_heads
    for layer in range(config.layers):
        prefix = f"{layer}."
        p = {k[len(prefix):]: v for k, v in parameters.items() if k.startswith(prefix)}

        def norm(value, gamma):
            return value / torch.sqrt(value.pow(2).mean(-1, keepdim=True) + config.rms_norm_eps) * gamma

        z = norm(x, p["attention_norm.weight"])
        b, s, h = z.shape
        q, k, v = (F.linear(z, p[f"attention.{n}_proj.weight"]).view(b, s, heads, h // heads).transpose(1, 2)
                   for n in ("q", "k", "v"))
        mixed = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        attn = F.linear(mixed.transpose(1, 2).reshape(b, s, h), p["attention.out_proj.weight"])
        x = x + attn
        z2 = norm(x, p["mlp_norm.weight"])
        gated = F.silu(F.linear(z2, p["mlp.gate_proj.weight"])) * F.linear(z2, p["mlp.up_proj.weight"])
        mlp = F.linear(gated, p["mlp.down_proj.weight"])
        x = x + mlp
        if sublayers is not None:
            sublayers.append({"attention_norm": z, "attention": attn, "mlp_norm": z2, "mlp": mlp})
        outputs.append(x)
    return outputs


def compare_tensor(name, actual, expected, *, atol=1e-6, rtol=1e-5):
    """Row describing the worst deviation; `ok` uses the allclose criterion."""
    actual, expected = actual.detach().double().cpu(), expected.detach().double().cpu()
    if actual.shape != expected.shape:
        return {"name": name, "ok": False, "reason": f"shape {tuple(actual.shape)} != {tuple(expected.shape)}"}
    diff = (actual - expected).abs()
    bound = atol + rtol * expected.abs()
    return {"name": name, "ok": bool((diff <= bound).all()), "max_abs": float(diff.max()) if diff.numel() else 0.0,
            "max_rel": float((diff / expected.abs().clamp_min(1e-30)).max()) if diff.numel() else 0.0}
