"""Checkpoint oracle: the same local Hugging Face checkpoint through the dense FP32 model and
through the shard runtime, one forward and one backward each, compared.

    python -m shardtrain_b200.utils.verify_checkpoint --checkpoint /path/to/qwen --hf-config /path/to/config.json
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 \
        -m shardtrain_b200.utils.verify_checkpoint --checkpoint DIR --hf-config FILE --fsdp 2

What the reference's `scripts/verify_qwen2_checkpoint.py:40-375` establishes, restated: the strict
reader accepts the files (names, shapes, tied aliases), the runtime's shards built straight from
the checkpoint reproduce the dense model's loss and every parameter gradient on a fixed token
batch, and nothing is updated (no optimizer exists; the one backward only retires the runtime's
units).  The report carries a digest of this rank's shards so two machines can compare what they
loaded.  Nothing is downloaded.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import tempfile

import torch


def shard_digest(runtime) -> str:
    """sha256 over this rank's FP32 shards in registry order (names included)."""
    h = hashlib.sha256()
    for name, handle in runtime.registry.items():
        h.update(name.encode())
        h.update(handle.local_shard.detach().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()


def worst(actual: torch.Tensor, expected: torch.Tensor) -> tuple[float, float]:
    diff = (actual.double() - expected.double()).abs()
    scale = expected.double().abs().max().clamp_min(1e-30)
    return float(diff.max()), float(diff.max() / scale)


def dense_oracle(model_config, checkpoint, batches):
    """Loss and gradients of the dense FP32 model over ALL data-parallel replicas' batches (equal
    sizes, so the global token mean is the mean of the per-batch means): what the runtime's
    globally normalised loss and reduced gradients must equal on every rank."""
    from shardtrain_b200.models.qwen2 import Qwen2CausalLM
    from shardtrain_b200.models.qwen2_checkpoint import load_qwen_checkpoint
    from shardtrain_b200.models.qwen2_factory import qwen_config_from

    model = Qwen2CausalLM(qwen_config_from(model_config))
    report = load_qwen_checkpoint(model, checkpoint)
    total = 0.0
    for ids in batches:
        out = model(ids, labels=ids)
        (out.loss / len(batches)).backward()
        total += float(out.loss.detach()) / len(batches)
    grads = {n: p.grad.detach().clone() for n, p in model.named_parameters()}
    return total, grads, report


def verify(config, checkpoint, *, batch: int, seed: int, atol: float, rtol: float) -> dict:
    from shardtrain_b200.launch.bootstrap import WorkerSession
    from shardtrain_b200.models.qwen2_factory import build_qwen_model
    from shardtrain_b200.runtime.engine import ShardedRuntime

    with WorkerSession(config, "runtime") as session:
        mesh = session.context
        batches = [torch.randint(config.model.vocab_size, (batch, config.model.seq_len),
                                 generator=torch.Generator().manual_seed(seed + replica))
                   for replica in range(config.parallel.fsdp_degree)]
        ids = batches[mesh.coordinate.fsdp]
        want_loss, want_grads, load_report = dense_oracle(config.model, checkpoint, batches)

        model = build_qwen_model(config.model, config.training.seed, checkpoint=checkpoint)
        runtime = ShardedRuntime(device=mesh.device, reshard_after_forward=True,
                                 communication_policy=config.runtime.communication_policy,
                                 diagnostics_enabled=False, compute_dtype="fp32",
                                 communication_backend="nccl" if mesh.device.type == "cuda" else "auto")
        runtime.register(model, mesh if session.worker.launched else None,
                         sp=config.parallel.sp_enabled)
        digest = shard_digest(runtime)
        device_ids = ids.to(mesh.device)
        with runtime.compute_context():
            runtime.zero_grad()
            runtime.qwen_global_seq = ids.shape[1]
            runtime.begin_step(runtime.step_id + 1)
            out = model(device_ids, labels=device_ids)
            out.loss.backward()
            runtime.finalize_backward()
            got_loss = float(runtime.qwen_reported_loss())
            runtime.end_step()
        problems = []
        if abs(got_loss - want_loss) > atol + rtol * abs(want_loss):
            problems.append(f"loss {got_loss!r} vs dense {want_loss!r}")
        worst_name, worst_abs, worst_rel = None, 0.0, 0.0
        if config.parallel.tp_degree == 1:
            # the reduced shard gradients, put together again, are the dense model's gradients
            for name, grad in runtime.reconstruct_tp_local(gradients=True).items():
                a, r = worst(grad.cpu(), want_grads[name])
                if r > worst_rel:
                    worst_name, worst_abs, worst_rel = name, a, r
                if a > atol + rtol * float(want_grads[name].abs().max()):
                    problems.append(f"gradient of {name}: max abs error {a:.3e}")
        if digest != shard_digest(runtime):
            problems.append("the shards changed although no optimizer exists")
        return {
            "checkpoint": load_report.checkpoint_path,
            "tensors_in_checkpoint": load_report.checkpoint_tensor_count,
            "omitted_tied_aliases": list(load_report.omitted_tied_aliases),
            "converted_dtypes": list(load_report.converted_dtypes),
            "parameters": sum(h.spec.numel for h in runtime.registry.values()),
            "rank": session.worker.rank, "mesh": config.parallel.strategy, "shard_sha256": digest,
            "loss_dense": want_loss, "loss_runtime": got_loss,
            "worst_gradient": {"name": worst_name, "max_abs": worst_abs, "relative_to_max": worst_rel},
            "passed": not problems, "problems": problems,
        }


def main(argv=None) -> int:
    from shardtrain_b200.config import config_from_dict
    from shardtrain_b200.models.qwen2 import Qwen2ModelConfig

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint", required=True, help="directory or .safetensors file")
    ap.add_argument("--hf-config", required=True, help="HF config.json / YAML of the model")
    ap.add_argument("--fsdp", type=int, default=1)
    ap.add_argument("--device", choices=["cpu", "cuda"], default="cpu")
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=16)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--atol", type=float, default=3e-6)
    ap.add_argument("--rtol", type=float, default=3e-5)
    args = ap.parse_args(argv)
    hf = Qwen2ModelConfig.from_file(args.hf_config)
    config = config_from_dict({
        "model": dict(model_type="qwen2", hf_config_path=str(args.hf_config), seq_len=args.seq_len,
                      vocab_size=hf.vocab_size, layers=hf.num_hidden_layers, hidden_size=hf.hidden_size,
                      num_heads=hf.num_attention_heads, num_key_value_heads=hf.num_key_value_heads,
                      mlp_hidden_size=hf.intermediate_size, rope_theta=hf.rope_theta,
                      rms_norm_eps=hf.rms_norm_eps, tie_word_embeddings=hf.tie_word_embeddings),
        "parallel": dict(fsdp_degree=args.fsdp, tp_degree=1, sp_enabled=False, device=args.device,
                         backend="nccl" if args.device == "cuda" else "gloo"),
        "runtime": dict(param_grouping="block", reshard_after_forward=True,
                        communication_policy="conservative"),
        "training": dict(dtype="fp32", optimizer="sgd", lr=1e-3, steps=1, local_batch_size=args.batch,
                         accumulation_steps=1, seed=args.seed),
        "debug": dict(output_dir=os.path.join(tempfile.gettempdir(), f"verify_checkpoint_{os.getpid()}"),
                      distributed_timeout_seconds=120),
    })
    report = verify(config, args.checkpoint, batch=args.batch, seed=args.seed, atol=args.atol,
                    rtol=args.rtol)
    print(json.dumps(report, indent=1))
    return 0 if report["passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
