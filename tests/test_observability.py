"""Rank logs, run metadata and the profile capture's bookkeeping (CPU)."""
import json
import logging

import pytest
import torch
import yaml

from shardtrain_b200.config import load_config
from shardtrain_b200.distributed.context import WorkerEnvironment
from shardtrain_b200.observability.logging import close_logger, make_rank_logger
from shardtrain_b200.observability.metadata import save_metadata, write_json
from shardtrain_b200.observability.profiling import ProfileCapture


def test_rank_logger_writes_json_lines_and_quiet_console_for_other_ranks(tmp_path, capsys):
    first, other = make_rank_logger(tmp_path, 0), make_rank_logger(tmp_path, 3)
    first.info("hello %d", 7)
    other.info("not on the console")
    try:
        raise ValueError("boom")
    except ValueError:
        other.exception("failed")
    close_logger(first)
    close_logger(other)
    err = capsys.readouterr().err
    assert "[rank 0] INFO hello 7" in err and "not on the console" not in err
    assert "[rank 3] ERROR failed" in err
    rows = [json.loads(line) for line in (tmp_path / "rank3.jsonl").read_text().splitlines()]
    assert [r["message"] for r in rows] == ["not on the console", "failed"]
    assert rows[1]["level"] == "ERROR" and "ValueError: boom" in rows[1]["exception"]
    assert all(r["rank"] == 3 and r["time_utc"].endswith("+00:00") for r in rows)
    assert not logging.getLogger("shardtrain.rank0").handlers


def test_metadata_files_describe_config_and_environment(tmp_path):
    config = load_config(None, ["--training.steps", "5", "--debug.output_dir", str(tmp_path)])
    worker = WorkerEnvironment.read({})
    save_metadata(tmp_path, config, worker, torch.device("cpu"))
    resolved = yaml.safe_load((tmp_path / "resolved_config.rank0.yaml").read_text())
    assert resolved["training"]["steps"] == 5 and resolved["parallel"]["fsdp_degree"] == 1
    env = json.loads((tmp_path / "environment.rank0.json").read_text())
    assert env["torch"] == torch.__version__ and env["device_name"] == "CPU"
    assert env["world_size"] == 1 and "sm_100a_extension" in env
    write_json(tmp_path / "x.json", {"a": torch.float32, "b": tmp_path})     # non-JSON values survive
    assert json.loads((tmp_path / "x.json").read_text())["a"] == "torch.float32"


def test_profile_capture_modes_on_cpu(tmp_path):
    with pytest.raises(ValueError):
        ProfileCapture(tmp_path, 0, "cpu", mode="bogus")
    with pytest.raises(ValueError):
        ProfileCapture(tmp_path, 0, "cpu", detail="bogus")
    off = ProfileCapture(tmp_path / "off", 0, "cpu", mode="off")
    off.start()
    off.step(1)
    off.close()
    assert not (tmp_path / "off").exists()
    capture = ProfileCapture(tmp_path / "torch", 1, "cpu", mode="torch")
    capture.start()
    torch.ones(8).sum()
    capture.step(1)
    capture.close()
    assert (tmp_path / "torch" / "profile.rank1.json").exists()
    record = json.loads((tmp_path / "torch" / "profiling.rank1.json").read_text())
    assert record["mode"] == "torch"


def test_worker_session_logs_bootstrap_and_worker_failures(tmp_path, monkeypatch):
    """A configuration that cannot run leaves "Worker bootstrap failed" in the rank log; an
    exception inside the session is logged as "Worker failed"; a malformed launcher environment
    still leaves a log behind."""
    from shardtrain_b200.config import ConfigError
    from shardtrain_b200.launch.bootstrap import WorkerSession

    for key in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(key, raising=False)
    bad = load_config(None, ["--parallel.fsdp_degree", "2", "--debug.output_dir", str(tmp_path / "bad")])
    with pytest.raises(ConfigError):
        with WorkerSession(bad, "runtime"):
            pass
    text = (tmp_path / "bad" / "rank0.jsonl").read_text()
    assert "Worker bootstrap failed" in text

    good = load_config(None, ["--debug.output_dir", str(tmp_path / "good")])
    with pytest.raises(RuntimeError, match="injected"):
        with WorkerSession(good, "train") as session:
            assert session.context.device.type == "cpu"
            raise RuntimeError("injected on the host")
    rows = [json.loads(line) for line in (tmp_path / "good" / "rank0.jsonl").read_text().splitlines()]
    assert any(r["message"] == "Worker failed" and "injected on the host" in r.get("exception", "")
               for r in rows)

    monkeypatch.setenv("RANK", "1")          # WORLD_SIZE missing: malformed launcher environment
    with pytest.raises(ConfigError):
        with WorkerSession(load_config(None, ["--debug.output_dir", str(tmp_path / "env")]), "train"):
            pass
    assert "Worker environment validation failed" in (tmp_path / "env" / "rank0.jsonl").read_text()
    with pytest.raises(ConfigError, match="output_dir"):
        WorkerSession(load_config(None, ["--debug.output_dir", " "]), "train")
