"""Run configuration: five YAML sections, frozen dataclasses, strict validation per mode.

The schema (section names, field names, defaults, override syntax `--section.field value`) is the
one of the reference's `src/sharded_runtime/config.py:17-268`, so its YAML presets load unchanged.
The validation rules are stated as a table of checks instead of a chain of `if`s.  Six optional
runtime fields are new and default to the reference behaviour: `communication_backend`
("auto" | "peer" | "nccl") selects the NVLink peer-memory kernels or the NCCL baseline path,
`retain_parameters` keeps the gathered compute-dtype parameters for the whole optimizer step,
`fused_allgather` ("auto" | "on" | "off") lets a decoder layer's forward GEMMs pull q|k|v and
gate|up from the owning ranks' shards instead of gathering them first, `wire_dtype`
("bf16" | "fp32") picks what the parameter gather moves over NVLink, and `fused_seq_gather`
lets the GEMM that consumes a sequence all-gather pull the peers' slices itself; `nvls`
("auto" | "off") allows the gradient reduce-scatter of FSDP-only meshes to run inside the NVSwitch;
`cuda_graphs` lets the sm_100a executor replay a decoder layer's launch sequence as one CUDA graph
once its arguments have repeated (FSDP-only meshes).

This module never imports torch.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any, Callable, get_type_hints

import yaml


class ConfigError(ValueError):
    """Raised for an invalid or unsupported configuration."""


@dataclass(frozen=True)
class ModelConfig:
    layers: int = 1
    hidden_size: int = 128
    num_heads: int = 4
    mlp_hidden_size: int = 256
    seq_len: int = 16
    dropout: float = 0.0
    rms_norm_eps: float = 1e-6
    model_type: str = "toy"
    hf_config_path: str = ""
    checkpoint_path: str = ""
    vocab_size: int = 128
    num_key_value_heads: int = 2
    rope_theta: float = 1000000.0
    tie_word_embeddings: bool = True


@dataclass(frozen=True)
class ParallelConfig:
    fsdp_degree: int = 1
    tp_degree: int = 1
    sp_enabled: bool = False
    device: str = "cpu"
    backend: str = "gloo"

    @property
    def world_size(self) -> int:
        return self.fsdp_degree * self.tp_degree

    @property
    def strategy(self) -> str:
        """`F{dp}T{tp}` name, with `/SP` when sequence parallelism is on."""
        return f"F{self.fsdp_degree}T{self.tp_degree}" + ("/SP" if self.sp_enabled else "")


@dataclass(frozen=True)
class RuntimeConfig:
    reshard_after_forward: bool = False
    materialization: str = "synchronous"
    prefetch: str = "none"
    param_grouping: str = "submodule"
    forward_prefetch: bool = False
    backward_prefetch: bool = False
    async_grad_rs: bool = False
    communication_policy: str = "conservative"
    communication_backend: str = "auto"
    retain_parameters: bool = False
    fused_allgather: str = "auto"
    wire_dtype: str = "bf16"
    fused_seq_gather: bool = False
    nvls: str = "off"
    cuda_graphs: bool = True


@dataclass(frozen=True)
class TrainingConfig:
    dtype: str = "fp32"
    optimizer: str = "sgd"
    lr: float = 0.001
    steps: int = 3
    local_batch_size: int = 2
    accumulation_steps: int = 1
    seed: int = 1234


@dataclass(frozen=True)
class DebugConfig:
    log_level: str = "INFO"
    distributed_timeout_seconds: int = 30
    output_dir: str = "runs/reference"


MODES = ("reference", "train", "smoke", "runtime")


def parse_strategy(name: str) -> tuple[int, int, bool]:
    """`"F4T2/SP"` -> (4, 2, True)."""
    text = name.strip().upper()
    sp = text.endswith("/SP")
    if sp:
        text = text[:-3]
    if not text.startswith("F") or "T" not in text:
        raise ConfigError(f"Strategy must look like F4T2 or F4T2/SP; got {name!r}")
    f, t = text[1:].split("T", 1)
    try:
        return int(f), int(t), sp
    except ValueError as exc:
        raise ConfigError(f"Strategy must look like F4T2 or F4T2/SP; got {name!r}") from exc


@dataclass(frozen=True)
class Config:
    model: ModelConfig = field(default_factory=ModelConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    runtime: RuntimeConfig = field(default_factory=RuntimeConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    debug: DebugConfig = field(default_factory=DebugConfig)

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)

    # ------------------------------------------------------------------ validation
    def _rules(self, world_size: int | None, mode: str) -> list[tuple[Callable[[], bool], str]]:
        m, p, r, t, d = self.model, self.parallel, self.runtime, self.training, self.debug
        qwen = m.model_type == "qwen2"
        runtime_mode = mode == "runtime"
        async_requested = (
            r.materialization != "synchronous"
            or r.prefetch != "none"
            or r.forward_prefetch
            or r.backward_prefetch
            or r.async_grad_rs
            or r.communication_policy != "conservative"
        )

        def finite_positive(x: Any) -> bool:
            return not isinstance(x, bool) and math.isfinite(x) and x > 0

        return [
            (lambda: m.model_type in {"toy", "qwen2"}, "model.model_type must be toy or qwen2"),
            (
                lambda: not qwen or mode in {"runtime", "smoke"},
                "Qwen2 training requires the ShardTrain runtime mode",
            ),
            (
                lambda: world_size is None or world_size == p.world_size,
                f"WORLD_SIZE={world_size} does not match fsdp_degree * tp_degree={p.world_size}",
            ),
            (
                lambda: m.hidden_size % m.num_heads == 0,
                "model.hidden_size must be divisible by model.num_heads",
            ),
            (
                lambda: m.hidden_size % p.tp_degree == 0,
                "model.hidden_size must be divisible by parallel.tp_degree",
            ),
            (
                lambda: m.num_heads % p.tp_degree == 0,
                "model.num_heads must be divisible by parallel.tp_degree",
            ),
            (
                lambda: m.mlp_hidden_size % p.tp_degree == 0,
                "model.mlp_hidden_size must be divisible by parallel.tp_degree",
            ),
            (
                lambda: not p.sp_enabled or p.tp_degree > 1,
                "SP requires parallel.tp_degree > 1; SP is not a mesh dimension",
            ),
            (
                lambda: not p.sp_enabled or m.seq_len % p.tp_degree == 0,
                "model.seq_len must be divisible by TP degree when SP is enabled",
            ),
            (
                lambda: p.device in {"cpu", "cuda"},
                "parallel.device must be cpu or cuda (index comes from LOCAL_RANK)",
            ),
            (lambda: p.backend in {"gloo", "nccl"}, "parallel.backend must be gloo or nccl"),
            (lambda: p.device != "cpu" or p.backend == "gloo", "CPU requires the Gloo backend"),
            (
                lambda: not (p.device == "cuda" and p.world_size > 1) or p.backend == "nccl",
                "Multi-process CUDA requires NCCL in the supported configuration",
            ),
            (lambda: m.dropout == 0.0, "Only dropout=0 is supported by the deterministic reference"),
            (lambda: finite_positive(m.rms_norm_eps), "model.rms_norm_eps must be finite and positive"),
            (lambda: finite_positive(t.lr), "training.lr must be finite and positive"),
            (
                lambda: type(t.seed) is int and 0 <= t.seed < 2**32,
                "training.seed must be an integer in [0, 2**32)",
            ),
            (
                lambda: not qwen
                or (t.dtype in {"fp32", "fp16", "bf16"} and t.optimizer in {"sgd", "adamw"}),
                "Qwen2 supports fp32/fp16/bf16 AMP with sgd/adamw",
            ),
            (
                lambda: not (qwen and t.dtype == "fp16") or p.device == "cuda",
                "Qwen2 fp16 AMP requires CUDA",
            ),
            (
                lambda: qwen or (t.dtype == "fp32" and t.optimizer == "sgd"),
                "M0/M1 support only FP32 with SGD",
            ),
            (
                lambda: not r.reshard_after_forward or runtime_mode,
                "reshard_after_forward is implemented in M3; set it to false for M0/M1",
            ),
            (
                lambda: runtime_mode or not async_requested,
                "Async materialization/prefetch is not implemented in M0/M1",
            ),
            (
                lambda: r.param_grouping == "submodule"
                or (runtime_mode and r.param_grouping == "block"),
                "Use param_grouping=block for runtime, submodule for the legacy path",
            ),
            (
                lambda: d.log_level in {"DEBUG", "INFO", "WARNING", "ERROR"},
                "debug.log_level must be DEBUG, INFO, WARNING or ERROR",
            ),
            (lambda: bool(d.output_dir.strip()), "debug.output_dir must not be empty"),
            (
                lambda: mode != "reference" or p.world_size == 1,
                "M0 reference training requires fsdp_degree=tp_degree=1; "
                "use --smoke-groups for topology/collective checks only",
            ),
            (
                lambda: mode != "train" or p.fsdp_degree == 1,
                "FSDP training is implemented in M2; M1 requires fsdp_degree=1",
            ),
            (
                lambda: mode != "train" or p.tp_degree in {1, 2},
                "M1 training supports only tp_degree=1 or 2",
            ),
            (
                lambda: not runtime_mode
                or r.communication_policy in {"conservative", "stream_ordered"},
                "communication_policy must be conservative or stream_ordered",
            ),
            (
                lambda: not runtime_mode
                or (p.fsdp_degree in {1, 2, 4, 8} and p.tp_degree in {1, 2, 4}),
                "v0.7 runtime supports F=1/2/4/8 and T=1/2/4",
            ),
            (
                lambda: not runtime_mode or t.accumulation_steps == 1 or qwen,
                "v0.7 runtime does not support microbatch gradient accumulation",
            ),
            (
                lambda: not runtime_mode or r.materialization == "synchronous",
                "Use independent async switches; keep materialization=synchronous",
            ),
            (
                lambda: not runtime_mode or r.prefetch == "none",
                "Use independent forward_prefetch/backward_prefetch flags",
            ),
            (
                lambda: r.communication_backend in {"auto", "peer", "nccl"},
                "runtime.communication_backend must be auto, peer or nccl",
            ),
            (
                lambda: r.communication_backend != "peer" or p.device == "cuda",
                "communication_backend=peer needs CUDA peer memory",
            ),
            (
                lambda: r.fused_allgather in {"auto", "on", "off"},
                "runtime.fused_allgather must be auto, on or off",
            ),
            (
                lambda: r.wire_dtype in {"bf16", "fp32"},
                "runtime.wire_dtype must be bf16 or fp32",
            ),
            (
                lambda: r.nvls in {"auto", "off"},
                "runtime.nvls must be auto or off",
            ),
        ]

    def validate(self, world_size: int | None = None, *, mode: str = "reference") -> None:
        if mode not in MODES:
            raise ConfigError(f"Unknown execution mode: {mode}")
        counts = {
            "model.layers": self.model.layers,
            "model.hidden_size": self.model.hidden_size,
            "model.num_heads": self.model.num_heads,
            "model.mlp_hidden_size": self.model.mlp_hidden_size,
            "model.seq_len": self.model.seq_len,
            "parallel.fsdp_degree": self.parallel.fsdp_degree,
            "parallel.tp_degree": self.parallel.tp_degree,
            "training.steps": self.training.steps,
            "training.local_batch_size": self.training.local_batch_size,
            "training.accumulation_steps": self.training.accumulation_steps,
            "debug.distributed_timeout_seconds": self.debug.distributed_timeout_seconds,
        }
        for name, value in counts.items():
            if type(value) is not int or value <= 0:
                raise ConfigError(f"{name} must be a positive integer; got {value!r}")
        for holds, message in self._rules(world_size, mode):
            if not holds():
                raise ConfigError(message)


_SECTIONS = {
    "model": ModelConfig,
    "parallel": ParallelConfig,
    "runtime": RuntimeConfig,
    "training": TrainingConfig,
    "debug": DebugConfig,
}


def _coerce(section: str, key: str, value: Any, expected: type) -> Any:
    if expected is float and type(value) in {int, float}:
        return float(value)
    if type(value) is not expected:
        raise ConfigError(f"{section}.{key} must be {expected.__name__}; got {value!r}")
    return value


def config_from_dict(data: dict[str, Any]) -> Config:
    if not isinstance(data, dict):
        raise ConfigError("Configuration root must be a mapping")
    extra = sorted(set(data) - set(_SECTIONS))
    if extra:
        raise ConfigError(f"Unknown config sections: {extra}")
    built = {}
    for name, cls in _SECTIONS.items():
        raw = data.get(name, {})
        if not isinstance(raw, dict):
            raise ConfigError(f"{name} must be a mapping")
        known = {f.name for f in fields(cls)}
        extra = sorted(set(raw) - known)
        if extra:
            raise ConfigError(f"Unknown fields in {name}: {extra}")
        hints = get_type_hints(cls)
        built[name] = cls(**{k: _coerce(name, k, v, hints[k]) for k, v in raw.items()})
    return Config(**built)


def load_config(filename: str | Path | None = None, overrides: list[str] | None = None) -> Config:
    """Read a YAML file, then apply `--section.field value` pairs (values parsed as YAML)."""
    try:
        data = yaml.safe_load(Path(filename).read_text(encoding="utf-8")) if filename else {}
    except (OSError, yaml.YAMLError) as exc:
        raise ConfigError(f"Cannot read configuration {filename}: {exc}") from exc
    # Keys and types of the file are checked before overrides so a typo is never hidden.
    resolved = config_from_dict(data or {}).to_dict()
    overrides = list(overrides or [])
    if len(overrides) % 2:
        raise ConfigError("Overrides require pairs: --section.field value")
    for flag, raw in zip(overrides[::2], overrides[1::2]):
        if not flag.startswith("--") or flag.count(".") != 1:
            raise ConfigError(f"Invalid override {flag!r}; expected --section.field value")
        section, key = flag[2:].split(".")
        if section not in resolved or key not in resolved[section]:
            raise ConfigError(f"Unknown config field: {flag}")
        try:
            resolved[section][key] = yaml.safe_load(raw)
        except yaml.YAMLError as exc:
            raise ConfigError(f"Invalid value for {flag}: {raw!r}") from exc
    return config_from_dict(resolved)


def with_strategy(config: Config, strategy: str) -> Config:
    """Return `config` with the parallel section set from an `F{dp}T{tp}[/SP]` name."""
    f, t, sp = parse_strategy(strategy)
    data = config.to_dict()
    data["parallel"].update(fsdp_degree=f, tp_degree=t, sp_enabled=sp)
    return config_from_dict(data)
