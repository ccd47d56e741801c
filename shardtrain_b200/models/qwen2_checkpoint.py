"""Local safetensors checkpoints: strict reading, slice reads, and writing.

The file format is parsed here directly (8-byte little-endian header length, JSON header with
`dtype/shape/data_offsets` per tensor, raw little-endian data), through a read-only memory map,
so a single row range of one tensor can be read without touching the rest of the file and without
an extra dependency.  `QwenCheckpoint` gives the same guarantees as the reference's reader
(`src/sharded_runtime/models/qwen2_checkpoint.py:45-283`): only local `.safetensors` files or a
`.index.json`, no pickle, no duplicate JSON keys, no shard outside the index directory, no tensor
hidden in a shard file that the index does not list, and an all-or-nothing `validate` of names,
shapes and tied aliases before any weight is copied.  `save_safetensors` is the writer used by
the full/sharded state-dict export (the reference has none).
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterator, Mapping

import torch
from torch import nn

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class CheckpointError(ValueError):
    """The checkpoint cannot be loaded without missing or ambiguous weights."""


@dataclass(frozen=True)
class CheckpointLoadReport:
    checkpoint_path: str
    checkpoint_tensor_count: int
    unique_tensor_count: int
    copied_bytes: int
    omitted_tied_aliases: tuple[str, ...]
    converted_dtypes: tuple[str, ...]


def _no_duplicate_keys(pairs: list[tuple[str, Any]]) -> dict[str, Any]:
    seen: dict[str, Any] = {}
    for key, value in pairs:
        if key in seen:
            raise CheckpointError(f"Duplicate JSON key in checkpoint index: {key}")
        seen[key] = value
    return seen


class SafetensorsFile:
    """Header of one `.safetensors` file plus mapped access to its tensors."""

    def __init__(self, path: Path) -> None:
        self.path = Path(path)
        try:
            with self.path.open("rb") as fh:
                (length,) = struct.unpack("<Q", fh.read(8))
                size = self.path.stat().st_size
                if length <= 0 or 8 + length > size:
                    raise CheckpointError(f"Corrupt safetensors header in {self.path}")
                header = json.loads(fh.read(length).decode("utf-8"), object_pairs_hook=_no_duplicate_keys)
        except CheckpointError:
            raise
        except Exception as exc:  # noqa: BLE001
            raise CheckpointError(f"Cannot inspect safetensors file {self.path}: {exc}") from exc
        self.data_start = 8 + length
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, dict[str, Any]] = {}
        for name, entry in header.items():
            dtype = entry.get("dtype")
            if dtype not in _DTYPES:
                raise CheckpointError(f"Unsupported dtype {dtype!r} for {name} in {self.path}")
            begin, end = entry["data_offsets"]
            shape = tuple(int(d) for d in entry["shape"])
            numel = 1
            for d in shape:
                numel *= d
            if end - begin != numel * _DTYPES[dtype].itemsize or self.data_start + end > size:
                raise CheckpointError(f"Inconsistent extent for {name} in {self.path}")
            self.entries[name] = {"dtype": _DTYPES[dtype], "shape": shape, "begin": begin, "end": end}

    def _view(self, name: str, first_row: int = 0, rows: int | None = None) -> torch.Tensor:
        entry = self.entries[name]
        shape, dtype = entry["shape"], entry["dtype"]
        row_elems = 1
        for d in shape[1:]:
            row_elems *= d
        total_rows = shape[0] if shape else 1
        rows = total_rows - first_row if rows is None else rows
        if first_row < 0 or rows < 0 or first_row + rows > total_rows:
            raise CheckpointError(f"Row range outside {name}")
        start = self.data_start + entry["begin"] + first_row * row_elems * dtype.itemsize
        nbytes = rows * row_elems * dtype.itemsize if shape else dtype.itemsize
        with self.path.open("rb") as fh, mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ) as mm:
            raw = bytearray(mm[start : start + nbytes])
        flat = torch.frombuffer(raw, dtype=dtype) if nbytes else torch.empty(0, dtype=dtype)
        return flat.reshape((rows, *shape[1:]) if shape else ())

    def tensor(self, name: str) -> torch.Tensor:
        return self._view(name)

    def rows(self, name: str, first_row: int, rows: int) -> torch.Tensor:
        return self._view(name, first_row, rows)


def save_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor],
                     metadata: Mapping[str, str] | None = None) -> None:
    """Write CPU tensors to one `.safetensors` file (names sorted, data 8-byte aligned)."""
    header: dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    blobs = []
    for name in order:
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise CheckpointError(f"Cannot serialise dtype {t.dtype} for {name}")
        blob = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * ((8 - len(encoded) % 8) % 8)
    target = Path(path)
    partial = target.with_suffix(target.suffix + ".partial")
    with partial.open("wb") as fh:
        fh.write(struct.pack("<Q", len(encoded)))
        fh.write(encoded)
        for blob in blobs:
            fh.write(blob)
    partial.replace(target)


class QwenCheckpoint:
    """Inspect a local HF checkpoint once, then hand out tensors (or row ranges) on demand."""

    def __init__(self, path: str | Path, expected_shapes: Mapping[str, tuple[int, ...]] | None = None,
                 tied_aliases: Mapping[str, str] | None = None) -> None:
        self.path = Path(path).expanduser().resolve()
        self._owner: dict[str, SafetensorsFile] = {}
        self._aliases: dict[str, str] = {}
        self._scan()
        if expected_shapes is not None:
            self.validate(expected_shapes, tied_aliases)
        elif tied_aliases:
            raise CheckpointError("tied_aliases require expected_shapes for validation")

    # ------------------------------------------------------------------ discovery
    def _entry_point(self) -> Path:
        if self.path.is_file():
            return self.path
        if not self.path.is_dir():
            raise CheckpointError(f"Checkpoint path does not exist: {self.path}")
        for name in ("model.safetensors.index.json", "model.safetensors"):
            if (self.path / name).is_file():
                return self.path / name
        loose = sorted(self.path.glob("*.safetensors"))
        if len(loose) != 1:
            raise CheckpointError(
                f"Expected model.safetensors or its index in {self.path}; "
                f"found {len(loose)} standalone safetensors files"
            )
        return loose[0]

    def _indexed_files(self, index: Path) -> dict[str, Path]:
        try:
            data = json.loads(index.read_text(encoding="utf-8"), object_pairs_hook=_no_duplicate_keys)
        except (OSError, json.JSONDecodeError) as exc:
            raise CheckpointError(f"Cannot read checkpoint index {index}: {exc}") from exc
        table = data.get("weight_map") if isinstance(data, dict) else None
        if not isinstance(table, dict):
            raise CheckpointError("Checkpoint index must contain a weight_map object")
        if not table:
            raise CheckpointError("Checkpoint weight_map must not be empty")
        root = index.parent.resolve()
        located: dict[str, Path] = {}
        for tensor_name, file_name in table.items():
            if not isinstance(tensor_name, str) or not isinstance(file_name, str):
                raise CheckpointError("Checkpoint weight_map keys and values must be strings")
            shard = (root / file_name).resolve()
            if not shard.is_relative_to(root):
                raise CheckpointError(f"Checkpoint shard escapes index directory: {file_name}")
            if shard.suffix != ".safetensors" or not shard.is_file():
                raise CheckpointError(f"Missing or unsupported checkpoint shard: {file_name}")
            located[tensor_name] = shard
        return located

    def _scan(self) -> None:
        entry = self._entry_point()
        listed: dict[str, Path] | None = None
        if entry.name.endswith(".index.json"):
            listed = self._indexed_files(entry)
            shard_paths = sorted(set(listed.values()))
        elif entry.suffix == ".safetensors":
            shard_paths = [entry]
        else:
            raise CheckpointError("Only local .safetensors files or .index.json are supported")
        for shard_path in shard_paths:
            shard = SafetensorsFile(shard_path)
            for name in shard.entries:
                if name in self._owner:
                    raise CheckpointError(f"Duplicate tensor across checkpoint shards: {name}")
                if listed is not None and listed.get(name) != shard_path:
                    raise CheckpointError(
                        f"Tensor {name} in {shard_path.name} is absent from the index "
                        "or mapped to a different shard"
                    )
                self._owner[name] = shard
        if not self._owner:
            raise CheckpointError("Checkpoint contains no tensors")
        if listed is not None:
            ghosts = sorted(set(listed) - self._owner.keys())
            if ghosts:
                raise CheckpointError(f"Index references absent tensors: {', '.join(ghosts)}")

    # ------------------------------------------------------------------ inspection
    @property
    def keys(self) -> tuple[str, ...]:
        return tuple(sorted(self._owner))

    @property
    def shapes(self) -> dict[str, tuple[int, ...]]:
        return {n: f.entries[n]["shape"] for n, f in self._owner.items()}

    @property
    def dtypes(self) -> dict[str, str]:
        return {n: _NAMES[f.entries[n]["dtype"]] for n, f in self._owner.items()}

    def validate(self, expected_shapes: Mapping[str, tuple[int, ...]],
                 tied_aliases: Mapping[str, str] | None = None) -> tuple[str, ...]:
        """Check every name and shape before anything is copied; returns the omitted aliases."""
        want = {n: tuple(s) for n, s in expected_shapes.items()}
        aliases = dict(tied_aliases or {})
        for alias, target in aliases.items():
            if alias == target or alias not in want or target not in want:
                raise CheckpointError(f"Invalid tied alias: {alias} -> {target}")
            if want[alias] != want[target] or target in aliases:
                raise CheckpointError(f"Inconsistent or chained tied alias: {alias} -> {target}")
        have = self.shapes
        problems = []
        missing = sorted(n for n in want if n not in have and aliases.get(n) not in have)
        if missing:
            problems.append("Missing keys: " + ", ".join(missing))
        extra = sorted(have.keys() - want.keys())
        if extra:
            problems.append("Unexpected keys: " + ", ".join(extra))
        wrong = [f"{n}: checkpoint {have[n]}, expected {s}" for n, s in want.items()
                 if n in have and have[n] != s]
        if wrong:
            problems.append("Shape mismatches: " + "; ".join(wrong))
        if problems:
            raise CheckpointError("Checkpoint validation failed. " + " | ".join(problems))
        for alias, target in aliases.items():
            if alias in have and target in have:
                if not torch.equal(self.get_tensor(alias), self.get_tensor(target)):
                    raise CheckpointError(f"Conflicting checkpoint values for tied keys: {target}, {alias}")
        self._aliases = aliases
        return tuple(sorted(a for a in aliases if a not in have))

    # ------------------------------------------------------------------ access
    def _resolve(self, name: str) -> str:
        if name in self._owner:
            return name
        target = self._aliases.get(name)
        if target in self._owner:
            return target
        raise CheckpointError(f"Checkpoint tensor not found: {name}")

    def get_tensor(self, name: str) -> torch.Tensor:
        name = self._resolve(name)
        return self._owner[name].tensor(name)

    def get_tensor_slice(self, name: str, index: Any) -> torch.Tensor:
        """Index a tensor reading only the needed leading-dimension rows where possible."""
        name = self._resolve(name)
        shard = self._owner[name]
        first = index[0] if isinstance(index, tuple) else index
        rows = shard.entries[name]["shape"][0] if shard.entries[name]["shape"] else 1
        if isinstance(first, slice) and first.step in (None, 1):
            start, stop, _ = first.indices(rows)
            part = shard.rows(name, start, max(0, stop - start))
            if isinstance(index, tuple) and len(index) > 1:
                return part[(slice(None), *index[1:])]
            return part
        return shard.tensor(name)[index]

    def iter_tensors(self, names: Iterator[str] | None = None) -> Iterator[tuple[str, torch.Tensor]]:
        for name in self.keys if names is None else names:
            yield name, self.get_tensor(name)


def iter_checkpoint_tensors(path: str | Path) -> Iterator[tuple[str, torch.Tensor]]:
    yield from QwenCheckpoint(path).iter_tensors()


def load_qwen_checkpoint(model: nn.Module, path: str | Path) -> CheckpointLoadReport:
    """Strict copy into an existing dense CPU model; tied keys are found by tensor identity."""
    targets = model.state_dict(keep_vars=True)
    if any(t.device.type != "cpu" for t in targets.values()):
        raise CheckpointError(
            "Dense checkpoint loading requires a CPU model; use QwenCheckpoint "
            "for memory-controlled direct shard registration"
        )
    first_name: dict[int, str] = {}
    aliases: dict[str, str] = {}
    for name, tensor in targets.items():
        if id(tensor) in first_name:
            aliases[name] = first_name[id(tensor)]
        else:
            first_name[id(tensor)] = name
    reader = QwenCheckpoint(path)
    omitted = reader.validate({n: tuple(t.shape) for n, t in targets.items()}, aliases)
    copied, converted = 0, []
    with torch.no_grad():
        for name, target in targets.items():
            if name in aliases:
                continue
            value = reader.get_tensor(name)
            if value.dtype != target.dtype:
                converted.append(name)
            target.copy_(value)
            copied += target.numel() * target.element_size()
    return CheckpointLoadReport(str(reader.path), len(reader.keys), len(first_name), copied,
                                omitted, tuple(converted))
