"""Multi-GPU checks of the sm_100a executor (run with -m gpu on a box with 2 or more GPUs; they
skip themselves on a single GPU).  Each case trains the small head_dim-128 Qwen2 for three steps
under torchrun and compares losses and reconstructed parameters with the dense model.  NVLS is
switched off for these child processes; the peer kernels use plain loads and stores."""
import json

import pytest
import torch

from tests.launch import run_workers

pytestmark = pytest.mark.gpu

COMMON = ["--device", "cuda", "--dtype", "bf16", "--optimizer", "sgd", "--flags", "111",
          "--policy", "stream_ordered", "--accum", 2]
CASES = [
    # name, ranks, mesh / model arguments
    ("fsdp2", 2, ["--fsdp", 2, "--shape", "d128"]),
    ("fsdp2_untied", 2, ["--fsdp", 2, "--shape", "d128", "--tied", 0]),
    ("tp2_sp", 2, ["--fsdp", 1, "--tp", 2, "--sp", 1, "--shape", "d128tp"]),
    ("tp2_sp_pulling_gemm", 2, ["--fsdp", 1, "--tp", 2, "--sp", 1, "--shape", "d128tp",
                                "--seq-pull", 1]),
    ("tp2", 2, ["--fsdp", 1, "--tp", 2, "--sp", 0, "--shape", "d128tp"]),
    ("fsdp2_tp2_sp", 4, ["--fsdp", 2, "--tp", 2, "--sp", 1, "--shape", "d128tp"]),
    ("fsdp2_tp2", 4, ["--fsdp", 2, "--tp", 2, "--sp", 0, "--shape", "d128tp", "--tied", 0]),
    ("fsdp4", 4, ["--fsdp", 4, "--shape", "d128"]),
    # q|k|v and gate|up pulled from the peers inside the forward GEMMs (fused all-gather -> GEMM)
    ("fsdp2_pull", 2, ["--fsdp", 2, "--shape", "d128", "--fused-allgather", "on"]),
    ("fsdp2_pull_fp32_wire", 2, ["--fsdp", 2, "--shape", "d128", "--fused-allgather", "on",
                                 "--wire", "fp32"]),
    # gradient reduce-scatter through the NVSwitch (multimem.ld_reduce); healthy run only
    ("fsdp2_nvls", 2, ["--fsdp", 2, "--shape", "d128", "--nvls", "auto"]),
    ("fsdp2_tp2_sp_pull", 4, ["--fsdp", 2, "--tp", 2, "--sp", 1, "--shape", "d128tp",
                              "--fused-allgather", "on", "--seq-pull", 1]),
]


@pytest.mark.parametrize("name,ranks,mesh", CASES, ids=[c[0] for c in CASES])
def test_fused_executor_matches_dense_on_a_mesh(tmp_path, name, ranks, mesh):
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    code, log = run_workers("tests.workers.qwen_worker", ranks, ["--out", tmp_path, *COMMON, *mesh],
                            timeout=300, env_extra={"NCCL_NVLS_ENABLE": "0"})
    assert code == 0, log[-3000:]
    for rank in range(ranks):
        record = json.loads((tmp_path / f"result.rank{rank}.json").read_text())
        assert record["shard_ok"] and record["live"] == 0
        assert record["param_err"] < 2e-4, record["errs"]
        for row in record["rows"]:
            assert abs(row["loss"] - row["ref"]) < 2e-3
        assert "fsdp_ag_cast" in record["kinds"]          # the peer-memory materialiser ran
        if "--nvls" in mesh and not record["nvls"]:
            pytest.skip(f"the fabric refused multicast: {record['nvls_refusal']}")
        if "--fused-allgather" in mesh:
            # the layers' forward gathers were partial: the GEMMs pulled the rest themselves
            assert record["kinds"].get("fsdp_ag_partial") == 3 * 2 * 2     # steps x micro x layers
