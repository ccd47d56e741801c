"""`shardtrain` command: train the configured model, or only check the process groups.

Same surface as the reference entry point (`src/sharded_runtime/train.py:9-122`): `--config`,
`--smoke-groups`, `--sharded-runtime`, and `--section.field value` overrides.  Routing:

* `--smoke-groups`            one collective per group of the mesh, results in `smoke.rank{r}.json`
* `model_type: qwen2`         the Qwen benchmark loop without warm-up (always the shard runtime)
* toy model, F > 1 or flag    shard runtime + `ShardedTrainer`, rows in `steps.rank{r}.json`
* toy model otherwise         FP32 reference or TP/SP `Trainer`, rows in `steps.rank{r}.json`
"""

from __future__ import annotations

import argparse
from dataclasses import asdict

from shardtrain_b200.config import ConfigError, load_config


def _smoke(config, session):
    from shardtrain_b200.observability.metadata import write_json

    results = session.context.smoke_collectives()
    write_json(session.directory / f"smoke.rank{session.worker.rank}.json", results)


def _runtime_rows(config, session):
    from shardtrain_b200.models.reference import build_reference_model, synthetic_batch
    from shardtrain_b200.runtime.engine import ShardedRuntime
    from shardtrain_b200.training.sharded_trainer import ShardedTrainer

    mesh, rc, tc = session.context, config.runtime, config.training
    model = build_reference_model(config.model, tc.seed)
    runtime = ShardedRuntime(
        device=mesh.device, reshard_after_forward=rc.reshard_after_forward,
        forward_prefetch=rc.forward_prefetch, backward_prefetch=rc.backward_prefetch,
        async_grad_rs=rc.async_grad_rs, communication_policy=rc.communication_policy,
        directory=session.directory, communication_backend=rc.communication_backend,
        retain_parameters=rc.retain_parameters, fused_allgather=rc.fused_allgather,
        wire_dtype=rc.wire_dtype, fused_seq_gather=rc.fused_seq_gather, nvls=rc.nvls, cuda_graphs=rc.cuda_graphs,
    )
    runtime.register(model, mesh, sp=config.parallel.sp_enabled)
    trainer = ShardedTrainer(model, runtime, tc.lr)
    rows = []
    for step in range(tc.steps):
        # every FSDP replica draws its own batch; the TP ranks of a replica share it
        seed = tc.seed + 100 * (step + 1) + mesh.coordinate.fsdp
        batch = synthetic_batch(config.model, tc.local_batch_size, seed, device=mesh.device)
        target = synthetic_batch(config.model, tc.local_batch_size, seed + 10000, device=mesh.device)
        result = trainer.train_step(runtime.input_for_rank(batch), runtime.input_for_rank(target))
        rows.append(asdict(result))
        session.logger.info("runtime step=%d loss=%.8f", result.step, result.loss)
    return rows


def _plain_rows(config, session):
    from shardtrain_b200.models.reference import build_reference_model, synthetic_batch
    from shardtrain_b200.parallel.model import parallelize_tp_sp
    from shardtrain_b200.training.trainer import Trainer

    mesh, tc = session.context, config.training
    model = build_reference_model(config.model, tc.seed).to(mesh.device)
    plan = None
    if config.parallel.tp_degree > 1:
        plan = parallelize_tp_sp(model, mesh.tp_group, sp=config.parallel.sp_enabled)
    trainer = Trainer(model, tc.lr, tc.accumulation_steps, tp_plan=plan)
    rows = []
    for step in range(tc.steps):
        # local_batch_size counts one micro-batch; a step consumes accumulation_steps of them
        batch = synthetic_batch(config.model, tc.local_batch_size * tc.accumulation_steps,
                                tc.seed + step + 1, device=mesh.device)
        if plan is not None:
            plan.group.broadcast(batch)
            batch = plan.input_for_rank(batch)
        result = trainer.train_step(batch)
        rows.append(asdict(result))
        session.logger.info("step=%d loss=%.8f gradient_l2=%.8f parameter_l2=%.8f", result.step,
                            result.loss, result.gradient_l2, result.parameter_l2)
    return rows


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(
        prog="shardtrain",
        description="shardtrain_b200: FP32 reference, TP/SP and FSDP shard-runtime training; "
                    "process-group smoke test",
        epilog="Config overrides: --section.field value (for example --training.steps 3)",
        allow_abbrev=False,
    )
    parser.add_argument("--config")
    parser.add_argument("--smoke-groups", action="store_true",
                        help="run one collective per process group and exit without training")
    parser.add_argument("--sharded-runtime", action="store_true",
                        help="train the toy model through the shard runtime even when F = 1")
    args, overrides = parser.parse_known_args(argv)
    try:
        config = load_config(args.config, overrides)
        if config.model.model_type == "qwen2" and not args.smoke_groups:
            from shardtrain_b200.training.qwen2_benchmark import run

            run(config, warmup=0, profile_mode="off")
            return 0
        # torch is imported only after the configuration has parsed
        from shardtrain_b200.launch.bootstrap import WorkerSession
        from shardtrain_b200.observability.metadata import write_json

        through_runtime = args.sharded_runtime or config.parallel.fsdp_degree > 1
        mode = "smoke" if args.smoke_groups else ("runtime" if through_runtime else "train")
        with WorkerSession(config, mode) as session:
            if args.smoke_groups:
                _smoke(config, session)
            else:
                rows = (_runtime_rows if through_runtime else _plain_rows)(config, session)
                write_json(session.directory / f"steps.rank{session.worker.rank}.json", rows)
    except ConfigError as exc:
        parser.error(str(exc))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
